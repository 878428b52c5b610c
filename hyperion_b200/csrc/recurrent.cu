// Kernels of mixers that carry a state from token to token instead of a cache of keys: the short
// causal convolution with its activation, the scan of a matrix-valued linear recurrence (the gated
// delta rule and the state-space recurrence of Mamba-2 are two modes of one kernel), and the gated
// group norm that follows it.  Everything here is float: inputs, state, decays, step sizes, gates
// of the recurrence, unit norms and sums.  A request's state lives in its slot of a per-request
// record (floats): first the matrices, then the convolution's last taps - 1 inputs.
//
// The scan.  Per head the state is a matrix S [n, e] (n: size of keys, e: size of values) and per
// token, with a key k, a query q (both of size n), a value v (size e), a decay a and a step b:
//     delta rule:   S <- a S;  u = b (v - S^T k);  S <- S + k u^T;  o = S^T q
//     state space:  S <- a S + k (b v)^T;                           o = S^T q + D v
//     retention:    S <- a S + k v^T  (a fixed per head);           o = S^T q
//     wkv:          o = S^T q + (sum_i u_i k_i q_i) v;  S <- diag(w) S + k v^T,  w_i = exp(-exp(x_i + w0_i))
//                   (a decay per key entry computed from the token, and a bonus u that only the current token gets)
//     channel delta: S <- diag(g) S;  u = b (v - S^T k);  S <- S + k u^T;  o = S^T q,  g_i = exp(-exp(A_log) softplus(x_i + bias_i))
//                   (the delta rule with a decay per key entry computed from the token)
// Column j of S (one value dimension) never meets another column, so the work is cut by columns:
// eight lanes share a column, each holding n / 8 of its entries in registers (groups of four
// consecutive entries, stored as S^T so that they are one 16-byte access), and a block of 128
// threads walks 16 columns through the tokens of one request's row in order.  Sums over n are
// taken in a fixed order (per lane in four chains, then a butterfly over the eight lanes), so a
// token's result does not depend on how the request was cut into steps or on what else is in
// the batch.
#include "common.cuh"

namespace {
constexpr int SCAN_THREADS = 128;
enum : int { MODE_DELTA = 0, MODE_STATE_SPACE = 1, MODE_RETENTION = 2, MODE_WKV = 3, MODE_CHANNEL_DELTA = 4 };

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---------------------------------------------------------------- causal convolution + SiLU
// out[t, c] = silu(bias[c] + sum_j weight[c, taps-1-j] * x[t-j, c]) over the tokens of t's own request; inputs before
// the row's first token come from the request's state (its last taps - 1 inputs, oldest first), which is zero for a new request.
__global__ void causal_conv_silu_kernel(const float* __restrict__ x, int x_stride, int col0, int channels, const float* __restrict__ weight,
                                        const float* __restrict__ bias, int taps, const float* __restrict__ state, size_t slot_stride,
                                        int state_off, const int* __restrict__ slots, const int* __restrict__ token_row,
                                        const int* __restrict__ row_start, float* __restrict__ out, int first_token) {
    const int t = first_token + blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;  // a block: one token, consecutive channels
    if (c >= channels) return;
    const int r = token_row[t];
    const int i = t - row_start[r];
    const float* kept = state + (size_t)slots[r] * slot_stride + state_off;
    float acc = bias ? bias[c] : 0.f;
    for (int j = taps - 1; j >= 0; --j) {  // oldest input first
        const float w = weight[(size_t)c * taps + taps - 1 - j];
        const float v = (i - j >= 0) ? x[(size_t)(t - j) * x_stride + col0 + c] : kept[(size_t)(taps - 1 + i - j) * channels + c];
        acc = fmaf(w, v, acc);
    }
    out[(size_t)t * channels + c] = silu_f(acc);
}

// The request's last taps - 1 inputs after this step's tokens (runs after the convolution has read the old ones).
__global__ void conv_state_update_kernel(const float* __restrict__ x, int x_stride, int col0, int channels, int taps, float* __restrict__ state,
                                         size_t slot_stride, int state_off, const int* __restrict__ slots, const int* __restrict__ row_start,
                                         int rows) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
    if (c >= channels || r >= rows) return;
    const int first = row_start[r], n = row_start[r + 1] - first, keep = taps - 1;
    float* kept = state + (size_t)slots[r] * slot_stride + state_off;
    for (int s = 0; s < keep; ++s) {  // ascending: an old entry is read (at s + n > s) before it is overwritten
        const int src = n - keep + s;
        kept[(size_t)s * channels + c] = src >= 0 ? x[(size_t)(first + src) * x_stride + col0 + c] : kept[(size_t)(s + n) * channels + c];
    }
}

// ---------------------------------------------------------------- the scan
struct ScanArgs {
    const float* k;      // [tokens, k_stride]: keys (convolved and activated where the mixer has a convolution), group g at g * n
    const float* q;      // [tokens, q_stride]: queries, likewise
    const float* v;      // [tokens, v_stride]: values, head h at h * e
    int k_stride, q_stride, v_stride;
    const float* proj;   // [tokens, proj_stride]: raw projections that give the decay and the step (wkv: heads * n entries at decay_off)
    int proj_stride, decay_off, step_off;
    const float* step;   // [tokens, step_stride]: the raw projection that gives the delta rule's step, head h at step_off + h (the modes whose step lies beside the decay: proj itself)
    int step_stride;
    const float* a_log;  // [heads] (wkv: w0 [heads * n])
    const float* dt_bias;  // [heads] (wkv: the bonus u [heads * n])
    const float* skip;   // [heads] (state space: D)
    float* state;
    size_t slot_stride;
    int state_off;
    const int* slots;
    const int* row_start;
    float* out;          // [tokens, heads * e], or null: only the states are wanted
    int heads, groups, n, n_padded, e;
    float q_scale;
};

template <int NG, int LPC, int CPT, int MODE>  // NG groups of four entries per lane, LPC lanes per column (n <= NG * 4 * LPC), CPT columns per thread
__global__ void __launch_bounds__(SCAN_THREADS) state_scan_kernel(const ScanArgs a) {
    // The tokens of the row pass through shared memory in chunks: while the block walks one chunk, every warp holds the next
    // chunk's share (every fourth token) in registers, already asked from memory; after the walk it turns them into what the
    // walk needs (unit keys and queries, decay, step) and writes them to the other buffer.  Nothing of that preparation lies on
    // the chain from one token's state to the next.  A thread owns its part of CPT columns: a token's key and query are read
    // from shared memory once for all of them, and the columns' chains, which never meet, fill one another's waits (a prompt
    // gives the GPU fewer warps than it has schedulers, so nothing else would).
    constexpr int NP = NG * 4 * LPC, NPR = NP / 32, GROUPS = 128 / LPC, COLUMNS = GROUPS * CPT, VR = (COLUMNS + 31) / 32;
    constexpr bool WKV = MODE == MODE_WKV, CHANNEL = MODE == MODE_CHANNEL_DELTA, DELTA = MODE == MODE_DELTA || CHANNEL;
    constexpr bool VEC = WKV || CHANNEL;  // a third vector per token (its decays) passes through shared memory: shorter chunks
    constexpr int CT = VEC ? (NP >= 256 ? 4 : (NP >= 128 ? 8 : 16)) : (NP >= 256 ? 8 : 16), PER_WARP = CT / 4;
    __shared__ __align__(16) float sk[2][CT][NP];
    __shared__ __align__(16) float sq[2][CT][NP];
    __shared__ __align__(16) float sw[VEC ? 2 : 1][VEC ? CT : 1][VEC ? NP : 4];
    __shared__ float sv[2][CT][VR * 32], sdecay[2][CT], sstep[2][CT];

    const int row = blockIdx.z, head = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int l = lane % LPC, cw = warp * (32 / LPC) + lane / LPC;  // this thread's columns: col0 + cw + GROUPS * c
    const int col0 = blockIdx.x * COLUMNS;
    const int t0 = a.row_start[row], t1 = a.row_start[row + 1];
    const int group = head / (a.heads / a.groups);
    float* const head_state = a.state + (size_t)a.slots[row] * a.slot_stride + a.state_off + (size_t)head * a.e * a.n_padded;

    float s[CPT][NG][4];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int col = col0 + cw + GROUPS * c;
#pragma unroll
        for (int r = 0; r < NG; ++r) {
            const int base = 4 * (LPC * r + l);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (col < a.e && base < a.n_padded) v = *reinterpret_cast<const float4*>(head_state + (size_t)col * a.n_padded + base);
            s[c][r][0] = v.x; s[c][r][1] = v.y; s[c][r][2] = v.z; s[c][r][3] = v.w;
        }
    }
    const float a_rate = (MODE == MODE_RETENTION || WKV) ? 0.f : expf(a.a_log[head]);
    const float fixed_decay = MODE == MODE_RETENTION ? a.a_log[head] : 0.f;
    const float bias = (MODE == MODE_RETENTION || VEC) ? 0.f : a.dt_bias[head];
    float w0[NPR], bonus[NPR];  // wkv: this lane's entries of the head's decay offset and bonus; channel delta: of the decay's bias
#pragma unroll
    for (int r = 0; r < NPR; ++r) {
        const int index = lane + 32 * r;
        w0[r] = (VEC && index < a.n) ? (WKV ? a.a_log : a.dt_bias)[(size_t)head * a.n + index] : 0.f;
        bonus[r] = (WKV && index < a.n) ? a.dt_bias[(size_t)head * a.n + index] : 0.f;
    }
    const float skip = MODE == MODE_STATE_SPACE ? a.skip[head] : 0.f;

    float pk[PER_WARP][NPR], pq[PER_WARP][NPR], pv[PER_WARP][VR], pdecay[PER_WARP], pstep[PER_WARP], pw[PER_WARP][VEC ? NPR : 1];
    auto prefetch = [&](int first) {
#pragma unroll
        for (int i = 0; i < PER_WARP; ++i) {
            const int t = first + warp + 4 * i;
            const bool live = t < t1;
            const size_t at = (size_t)(live ? t : t0);
            const float* k = a.k + at * a.k_stride + (size_t)group * a.n;
            const float* q = a.q + at * a.q_stride + (size_t)group * a.n;
            const float* vals = a.v + at * a.v_stride + (size_t)head * a.e;
#pragma unroll
            for (int r = 0; r < NPR; ++r) {
                const int index = lane + 32 * r;
                pk[i][r] = (live && index < a.n) ? k[index] : 0.f;
                pq[i][r] = (live && index < a.n) ? q[index] : 0.f;
            }
#pragma unroll
            for (int r = 0; r < VR; ++r) {
                const int column = lane + 32 * r;
                pv[i][r] = (live && column < COLUMNS && col0 + column < a.e) ? vals[col0 + column] : 0.f;
            }
            const float* p = a.proj + at * a.proj_stride;
            if (VEC) {
#pragma unroll
                for (int r = 0; r < NPR; ++r) {
                    const int index = lane + 32 * r;
                    pw[i][r] = (live && index < a.n) ? p[a.decay_off + (size_t)head * a.n + index] : 0.f;
                }
            }
            pdecay[i] = (live && MODE != MODE_RETENTION && !VEC) ? p[a.decay_off + head] : 0.f;
            pstep[i] = (live && DELTA) ? a.step[at * a.step_stride + a.step_off + head] : 0.f;
        }
    };
    auto publish = [&](int buffer) {
#pragma unroll
        for (int i = 0; i < PER_WARP; ++i) {
            const int j = warp + 4 * i;
            float ik = 1.f, iq = 1.f;
            if (DELTA) {  // keys and queries become unit vectors; the query also takes the scale
                float sum_k = 0.f, sum_q = 0.f;
#pragma unroll
                for (int r = 0; r < NPR; ++r) { sum_k = fmaf(pk[i][r], pk[i][r], sum_k); sum_q = fmaf(pq[i][r], pq[i][r], sum_q); }
                ik = 1.0f / sqrtf(warp_sum(sum_k) + 1e-6f);
                iq = a.q_scale / sqrtf(warp_sum(sum_q) + 1e-6f);
            }
#pragma unroll
            for (int r = 0; r < NPR; ++r) {
                sk[buffer][j][lane + 32 * r] = pk[i][r] * ik;
                sq[buffer][j][lane + 32 * r] = pq[i][r] * iq;
            }
#pragma unroll
            for (int r = 0; r < VR; ++r) sv[buffer][j][lane + 32 * r] = pv[i][r];
            float bonus_dot = 0.f;
            if (WKV) {  // the entries' decays, and what the bonus adds to the token's own value: sum_i u_i k_i q_i
#pragma unroll
                for (int r = 0; r < NPR; ++r) {
                    sw[buffer][j][lane + 32 * r] = expf(-expf(pw[i][r] + w0[r]));
                    bonus_dot = fmaf(bonus[r] * pk[i][r], pq[i][r], bonus_dot);
                }
                bonus_dot = warp_sum(bonus_dot);
            }
            if (CHANNEL) {  // the entries' decays
#pragma unroll
                for (int r = 0; r < NPR; ++r) sw[buffer][j][lane + 32 * r] = expf(-a_rate * softplus_f(pw[i][r] + w0[r]));
            }
            if (lane == 0) {
                float decay, step;
                if (WKV) {
                    decay = 1.f;
                    step = bonus_dot;
                } else if (CHANNEL) {
                    decay = 1.f;
                    step = 1.0f / (1.0f + expf(-pstep[i]));
                } else if (MODE == MODE_DELTA) {
                    decay = expf(-a_rate * softplus_f(pdecay[i] + bias));
                    step = 1.0f / (1.0f + expf(-pstep[i]));
                } else if (MODE == MODE_RETENTION) {  // the head's decay is a constant of the model; keys enter as they are
                    decay = fixed_decay;
                    step = 1.f;
                } else {
                    step = softplus_f(pdecay[i] + bias);
                    decay = expf(-a_rate * step);
                }
                sdecay[buffer][j] = decay;
                sstep[buffer][j] = step;
            }
        }
    };

    prefetch(t0);
    publish(0);
    __syncthreads();
    int buffer = 0;
    for (int first = t0; first < t1; first += CT, buffer ^= 1) {
        const bool more = first + CT < t1;
        if (more) prefetch(first + CT);  // in flight while this chunk is walked
        const int count = min(CT, t1 - first);
        for (int j = 0; j < count; ++j) {
            const float decay = sdecay[buffer][j], step = sstep[buffer][j];
            float ck[NG][4], cq[NG][4];
#pragma unroll
            for (int r = 0; r < NG; ++r) {
                const float4 k4 = *reinterpret_cast<const float4*>(&sk[buffer][j][4 * (LPC * r + l)]);
                const float4 q4 = *reinterpret_cast<const float4*>(&sq[buffer][j][4 * (LPC * r + l)]);
                ck[r][0] = k4.x; ck[r][1] = k4.y; ck[r][2] = k4.z; ck[r][3] = k4.w;
                cq[r][0] = q4.x; cq[r][1] = q4.y; cq[r][2] = q4.z; cq[r][3] = q4.w;
            }
            float cv[CPT], u[CPT], o[CPT];
#pragma unroll
            for (int c = 0; c < CPT; ++c) cv[c] = sv[buffer][j][cw + GROUPS * c];
            float cd[VEC ? NG : 1][4];
            if (VEC) {
#pragma unroll
                for (int r = 0; r < NG; ++r) {
                    const float4 d4 = *reinterpret_cast<const float4*>(&sw[buffer][j][4 * (LPC * r + l)]);
                    cd[r][0] = d4.x; cd[r][1] = d4.y; cd[r][2] = d4.z; cd[r][3] = d4.w;
                }
            }
            if (WKV) {
#pragma unroll
                for (int c = 0; c < CPT; ++c) {  // the query meets the state as the token found it; then the state fades and takes k v^T
                    float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int r = 0; r < NG; ++r)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            part[i] = fmaf(s[c][r][i], cq[r][i], part[i]);
                            s[c][r][i] = fmaf(s[c][r][i], cd[r][i], ck[r][i] * cv[c]);
                        }
                    o[c] = (part[0] + part[1]) + (part[2] + part[3]);
                }
#pragma unroll
                for (int offset = 1; offset < LPC; offset <<= 1)
#pragma unroll
                    for (int c = 0; c < CPT; ++c) o[c] += __shfl_xor_sync(0xffffffffu, o[c], offset);
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
                    const int col = col0 + cw + GROUPS * c;
                    if (l == 0 && col < a.e && a.out) a.out[((size_t)(first + j) * a.heads + head) * a.e + col] = fmaf(step, cv[c], o[c]);
                }
                continue;
            }
            if (DELTA) {
                float dot[CPT];
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
                    float part[4] = {0.f, 0.f, 0.f, 0.f};  // four chains instead of one: the sum's order is fixed all the same
#pragma unroll
                    for (int r = 0; r < NG; ++r)
#pragma unroll
                        for (int i = 0; i < 4; ++i) { s[c][r][i] *= CHANNEL ? cd[CHANNEL ? r : 0][i] : decay; part[i] = fmaf(s[c][r][i], ck[r][i], part[i]); }
                    dot[c] = (part[0] + part[1]) + (part[2] + part[3]);
                }
#pragma unroll
                for (int offset = 1; offset < LPC; offset <<= 1)
#pragma unroll
                    for (int c = 0; c < CPT; ++c) dot[c] += __shfl_xor_sync(0xffffffffu, dot[c], offset);
#pragma unroll
                for (int c = 0; c < CPT; ++c) u[c] = step * (cv[c] - dot[c]);
            } else {
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
#pragma unroll
                    for (int r = 0; r < NG; ++r)
#pragma unroll
                        for (int i = 0; i < 4; ++i) s[c][r][i] *= decay;
                    u[c] = step * cv[c];
                }
            }
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int r = 0; r < NG; ++r)
#pragma unroll
                    for (int i = 0; i < 4; ++i) { s[c][r][i] = fmaf(ck[r][i], u[c], s[c][r][i]); part[i] = fmaf(s[c][r][i], cq[r][i], part[i]); }
                o[c] = (part[0] + part[1]) + (part[2] + part[3]);
            }
#pragma unroll
            for (int offset = 1; offset < LPC; offset <<= 1)
#pragma unroll
                for (int c = 0; c < CPT; ++c) o[c] += __shfl_xor_sync(0xffffffffu, o[c], offset);
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const int col = col0 + cw + GROUPS * c;
                const float out = MODE == MODE_STATE_SPACE ? fmaf(skip, cv[c], o[c]) : o[c];
                if (l == 0 && col < a.e && a.out) a.out[((size_t)(first + j) * a.heads + head) * a.e + col] = out;
            }
        }
        if (!more) break;
        publish(buffer ^ 1);
        __syncthreads();
    }
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int col = col0 + cw + GROUPS * c;
#pragma unroll
        for (int r = 0; r < NG; ++r) {
            const int base = 4 * (LPC * r + l);
            if (col < a.e && base < a.n_padded)
                *reinterpret_cast<float4*>(head_state + (size_t)col * a.n_padded + base) = make_float4(s[c][r][0], s[c][r][1], s[c][r][2], s[c][r][3]);
        }
    }
}

template <int MODE>
int launch_scan(const ScanArgs& a, int rows, cudaStream_t stream) {
    // Eight lanes per column; one column per thread for the delta rule, two for the state-space recurrence, whatever the batch (a
    // token's sums must not change with it).  Measured on a B200 at heads x e = 2,048 and 4,096 with n = 128, a prompt of 2,048
    // tokens: sixteen or thirty-two lanes per column (more warps, fewer entries each) took 1.3 to 2 times as long, because every
    // warp reads the whole key and query of every token whatever it owns of the state.  More columns per thread go the other way:
    // the state-space scan fell from 668 / 944 us to 498 / 660 us with two (986 with four), the delta rule, whose columns each add a
    // reduction to the chain, rose from 783 / 939 us to 960 with two and 1,071 with four; eight decoded tokens gain a fifth either way.
    constexpr int LANES = 8;
    const int per_lane = (a.n_padded + 4 * LANES - 1) / (4 * LANES);  // groups of four entries per lane
    constexpr int PER_THREAD = (MODE == MODE_DELTA || MODE == MODE_CHANNEL_DELTA) ? 1 : 2;  // wkv: two, like the other recurrences whose columns add no reduction to the chain
    const int columns = (128 / LANES) * PER_THREAD;
    const dim3 grid((a.e + columns - 1) / columns, a.heads, rows);
    if (per_lane <= 1) state_scan_kernel<1, LANES, PER_THREAD, MODE><<<grid, SCAN_THREADS, 0, stream>>>(a);
    else if (per_lane <= 2) state_scan_kernel<2, LANES, PER_THREAD, MODE><<<grid, SCAN_THREADS, 0, stream>>>(a);
    else if (per_lane <= 4) state_scan_kernel<4, LANES, PER_THREAD, MODE><<<grid, SCAN_THREADS, 0, stream>>>(a);
    else state_scan_kernel<8, LANES, PER_THREAD, MODE><<<grid, SCAN_THREADS, 0, stream>>>(a);
    return launch_status();
}

// ---------------------------------------------------------------- gated group norm
// One block per (token, group of `group` columns).  gate_first: v = y * silu(g), out = v / rms(v) * w; otherwise
// out = y / rms(y) * w * silu(g); with sigmoid_gate the gate is sigmoid(g) instead of silu(g).  The weight has `weight_len` entries and is indexed by column % weight_len (a weight
// of one head's size is shared by all heads; no weight at all: a plain unit RMS).  `scale` multiplies the result before its one rounding.
__device__ __forceinline__ float gate_f(float z, int sigmoid_gate) { return sigmoid_gate ? 1.0f / (1.0f + expf(-z)) : silu_f(z); }

template <typename TO>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, int y_stride, const float* __restrict__ gate, int gate_stride,
                                        int gate_off, const float* __restrict__ weight, int weight_len, int group, int gate_first,
                                        float eps, float scale, TO* __restrict__ out, int out_stride, int sigmoid_gate) {
    __shared__ float scratch[32];
    const int t = blockIdx.x, first = blockIdx.y * group;
    const float* yrow = y + (size_t)t * y_stride + first;
    const float* grow = gate + (size_t)t * gate_stride + gate_off + first;
    float sum = 0.f;
    for (int j = threadIdx.x; j < group; j += blockDim.x) {
        float v = yrow[j];
        if (gate_first) v *= gate_f(grow[j], sigmoid_gate);
        sum = fmaf(v, v, sum);
    }
    const float inv = 1.0f / sqrtf(block_sum(sum, scratch) / (float)group + eps);
    for (int j = threadIdx.x; j < group; j += blockDim.x) {
        const float g = gate_f(grow[j], sigmoid_gate);
        float v = yrow[j];
        if (gate_first) v *= g;
        v = v * inv * (weight ? weight[(first + j) % weight_len] : 1.f);
        if (!gate_first) v *= g;
        out[(size_t)t * out_stride + first + j] = from_float<TO>(v * scale);
    }
}

// The same for groups of up to 1,024 columns: a warp per (token, group), four of them in a block; the lanes' partial sums
// meet in a butterfly of fixed shape.
template <typename TO>
__global__ void gated_group_norm_warp_kernel(const float* __restrict__ y, int y_stride, const float* __restrict__ gate, int gate_stride,
                                             int gate_off, const float* __restrict__ weight, int weight_len, int group, int groups, int gate_first,
                                             float eps, float scale, TO* __restrict__ out, int out_stride, int sigmoid_gate) {
    const int t = blockIdx.x, which = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (which >= groups) return;
    const int first = which * group;
    const float* yrow = y + (size_t)t * y_stride + first;
    const float* grow = gate + (size_t)t * gate_stride + gate_off + first;
    float sum = 0.f;
    for (int j = lane; j < group; j += 32) {
        float v = yrow[j];
        if (gate_first) v *= gate_f(grow[j], sigmoid_gate);
        sum = fmaf(v, v, sum);
    }
    const float inv = 1.0f / sqrtf(warp_sum(sum) / (float)group + eps);
    for (int j = lane; j < group; j += 32) {
        const float g = gate_f(grow[j], sigmoid_gate);
        float v = yrow[j];
        if (gate_first) v *= g;
        v = v * inv * (weight ? weight[(first + j) % weight_len] : 1.f);
        if (!gate_first) v *= g;
        out[(size_t)t * out_stride + first + j] = from_float<TO>(v * scale);
    }
}
}  // namespace

HB_EXPORT int hb_causal_conv_silu(const float* x, int x_stride, int col0, int channels, const float* weight, const float* bias, int taps,
                                  const float* state, long long slot_stride, int state_off, const int* slots, const int* token_row,
                                  const int* row_start, float* out, int tokens, cudaStream_t stream) {
    if (tokens <= 0 || channels <= 0) return 0;
    if (taps < 1) return HB_BAD_ARGUMENT;
    for (int first = 0; first < tokens; first += 65535) {  // the grid's second dimension holds 65,535 tokens
        const int count = tokens - first < 65535 ? tokens - first : 65535;
        causal_conv_silu_kernel<<<dim3((channels + 255) / 256, count), 256, 0, stream>>>(x, x_stride, col0, channels, weight, bias, taps, state, (size_t)slot_stride,
                                                                                        state_off, slots, token_row, row_start, out, first);
    }
    return launch_status();
}

HB_EXPORT int hb_conv_state_update(const float* x, int x_stride, int col0, int channels, int taps, float* state, long long slot_stride,
                                   int state_off, const int* slots, const int* row_start, int rows, cudaStream_t stream) {
    if (rows <= 0 || channels <= 0 || taps <= 1) return 0;
    if (rows > 65535) return HB_UNSUPPORTED_SIZE;
    conv_state_update_kernel<<<dim3((channels + 127) / 128, rows), 128, 0, stream>>>(x, x_stride, col0, channels, taps, state, (size_t)slot_stride,
                                                                                     state_off, slots, row_start, rows);
    return launch_status();
}

// mode 2: retention (decay = a_log[head] itself, a constant of the model; step = 1; keys, queries and values as given; proj, dt_bias and skip unused).
// mode 0: gated delta rule (keys and queries made unit vectors, q times q_scale; decay = exp(-exp(a_log) softplus(proj[decay_off] + dt_bias)),
// step = sigmoid(proj[step_off])).  mode 1: state space (step = softplus(proj[decay_off] + dt_bias), decay = exp(-exp(a_log) step), skip = D).
// The state of (slot, head) is S^T [e, n_padded] at state + slot * slot_stride + state_off; n_padded, state_off and slot_stride are multiples of 4.
HB_EXPORT int hb_state_scan(int mode, const float* conv, int conv_stride, int k_off, int q_off, int v_off, const float* proj, int proj_stride,
                            int decay_off, int step_off, const float* a_log, const float* dt_bias, const float* skip, float* state,
                            long long slot_stride, int state_off, const int* slots, const int* row_start, float* out, int rows, int heads,
                            int groups, int n, int n_padded, int e, float q_scale, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (n <= 0 || n > 256 || e <= 0 || heads <= 0 || groups <= 0 || heads % groups || rows > 65535 || heads > 65535) return HB_UNSUPPORTED_SIZE;
    if (n_padded < n || (n_padded & 3) || (state_off & 3) || (slot_stride & 3) || (((uintptr_t)state) & 15)) return HB_BAD_ARGUMENT;
    ScanArgs a{conv + k_off, conv + q_off, conv + v_off, conv_stride, conv_stride, conv_stride, proj, proj_stride, decay_off, step_off, proj, proj_stride, a_log, dt_bias, skip,
               state, (size_t)slot_stride, state_off, slots, row_start, out, heads, groups, n, n_padded, e, q_scale};
    if (mode == MODE_DELTA) return launch_scan<MODE_DELTA>(a, rows, stream);
    if (mode == MODE_STATE_SPACE) return launch_scan<MODE_STATE_SPACE>(a, rows, stream);
    if (mode == MODE_RETENTION) return launch_scan<MODE_RETENTION>(a, rows, stream);
    return HB_BAD_ARGUMENT;
}

// The delta rule with a decay per key entry (see the head of this file): keys, queries and values at k_off, q_off and v_off of `conv`
// (groups * n, groups * n and heads * e columns), the decays' pre-activations in `decay` [tokens, heads * n] with their bias
// dt_bias [heads * n] and the rate a_log [heads], the step's pre-activation (one per head) at step_off of `step`.  The state as in hb_state_scan.
HB_EXPORT int hb_channel_delta_scan(const float* conv, int conv_stride, int k_off, int q_off, int v_off, const float* decay, int decay_stride, int decay_off,
                                    const float* step, int step_stride, int step_off, const float* a_log, const float* dt_bias, float* state,
                                    long long slot_stride, int state_off, const int* slots, const int* row_start, float* out, int rows, int heads,
                                    int groups, int n, int n_padded, int e, float q_scale, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (n <= 0 || n > 256 || e <= 0 || heads <= 0 || groups <= 0 || heads % groups || rows > 65535 || heads > 65535) return HB_UNSUPPORTED_SIZE;
    if (n_padded < n || (n_padded & 3) || (state_off & 3) || (slot_stride & 3) || (((uintptr_t)state) & 15) || !a_log || !dt_bias) return HB_BAD_ARGUMENT;
    ScanArgs a{conv + k_off, conv + q_off, conv + v_off, conv_stride, conv_stride, conv_stride, decay, decay_stride, decay_off, step_off, step, step_stride,
               a_log, dt_bias, nullptr, state, (size_t)slot_stride, state_off, slots, row_start, out, heads, groups, n, n_padded, e, q_scale};
    return launch_scan<MODE_CHANNEL_DELTA>(a, rows, stream);
}

// The wkv recurrence: keys, queries and values from three float matrices of their own (heads * n, heads * n and heads * e columns), the
// decays' pre-activations x [tokens, heads * n] (w = exp(-exp(x + w0))), w0 and the bonus u [heads * n].  The state as in hb_state_scan.
HB_EXPORT int hb_wkv_scan(const float* k, int k_stride, const float* q, int q_stride, const float* v, int v_stride, const float* x, int x_stride, int x_off,
                          const float* w0, const float* bonus, float* state, long long slot_stride, int state_off, const int* slots, const int* row_start,
                          float* out, int rows, int heads, int n, int n_padded, int e, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (n <= 0 || n > 256 || e <= 0 || heads <= 0 || rows > 65535 || heads > 65535) return HB_UNSUPPORTED_SIZE;
    if (n_padded < n || (n_padded & 3) || (state_off & 3) || (slot_stride & 3) || (((uintptr_t)state) & 15) || !w0 || !bonus) return HB_BAD_ARGUMENT;
    ScanArgs a{k, q, v, k_stride, q_stride, v_stride, x, x_stride, x_off, 0, x, x_stride, w0, bonus, nullptr, state, (size_t)slot_stride, state_off, slots, row_start, out,
               heads, heads, n, n_padded, e, 1.f};
    return launch_scan<MODE_WKV>(a, rows, stream);
}

// ---------------------------------------------------------------- token shift
// A mixer that reads every token beside the one before it: input s of the mixer is h + (h' - h) * mu_s, h' being the row of the token
// before (of the same request; its last token of the step before, kept in the request's slot, for the first token of a step; zeros
// at the start of a request, which is what a fresh slot holds).  out [n_mix, tokens, hidden]: a dense matrix per input.  The
// arithmetic is float, rounded once.  hb_token_shift_keep then stores every row's last token (as floats) for the next step.
namespace {
template <typename T>
__global__ void token_shift_mix_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ mu, int n_mix, const float* __restrict__ state,
                                       size_t slot_stride, int state_off, const int* __restrict__ slots, const int* __restrict__ token_row,
                                       const int* __restrict__ row_start, T* __restrict__ out, int tokens, int hidden) {
    const int t = blockIdx.x;
    const int row = token_row[t];
    const bool first = t == row_start[row];
    const T* now = x + (size_t)t * x_stride;
    const T* before = x + (size_t)(t - 1) * x_stride;
    const float* kept = state + (size_t)slots[row] * slot_stride + state_off;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float h = to_float(now[i]);
        const float d = (first ? kept[i] : to_float(before[i])) - h;
        for (int m = 0; m < n_mix; ++m) out[((size_t)m * tokens + t) * hidden + i] = from_float<T>(fmaf(d, mu[(size_t)m * hidden + i], h));
    }
}

// Four columns per access, for rows of a multiple of four columns that start on 16-byte boundaries.
template <typename T>
__global__ void token_shift_mix4_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ mu, int n_mix, const float* __restrict__ state,
                                        size_t slot_stride, int state_off, const int* __restrict__ slots, const int* __restrict__ token_row,
                                        const int* __restrict__ row_start, T* __restrict__ out, int tokens, int hidden) {
    const int t = blockIdx.x;
    const int row = token_row[t];
    const bool first = t == row_start[row];
    const T* now = x + (size_t)t * x_stride;
    const T* before = x + (size_t)(t - 1) * x_stride;
    const float* kept = state + (size_t)slots[row] * slot_stride + state_off;
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
        float h[4], d[4];
        load4(now + i, h);
        if (first) load4(kept + i, d);
        else load4(before + i, d);
#pragma unroll
        for (int e = 0; e < 4; ++e) d[e] -= h[e];
        for (int m = 0; m < n_mix; ++m) {
            float w[4], v[4];
            load4(mu + (size_t)m * hidden + i, w);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = fmaf(d[e], w[e], h[e]);
            store4(out + ((size_t)m * tokens + t) * hidden + i, v);
        }
    }
}

template <typename T>
__global__ void token_shift_keep_kernel(const T* __restrict__ x, int x_stride, float* __restrict__ state, size_t slot_stride, int state_off,
                                        const int* __restrict__ slots, const int* __restrict__ row_start, int hidden) {
    const int row = blockIdx.x;
    const int last = row_start[row + 1] - 1;
    if (last < row_start[row]) return;
    float* kept = state + (size_t)slots[row] * slot_stride + state_off;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) kept[i] = to_float(x[(size_t)last * x_stride + i]);
}

template <typename T>
__global__ void tanh_rows_kernel(const float* __restrict__ x, T* __restrict__ out, long long count) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) out[i] = from_float<T>(tanhf(x[i]));
}
}  // namespace

HB_EXPORT int hb_token_shift_mix(const void* x, int is_bf16, int x_stride, const float* mu, int n_mix, const float* state, long long slot_stride, int state_off,
                                 const int* slots, const int* token_row, const int* row_start, void* out, int tokens, int hidden, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (hidden <= 0 || n_mix <= 0) return HB_UNSUPPORTED_SIZE;
    const int threads = hidden >= 1024 ? 256 : 128;
    const bool by_four = hidden % 4 == 0 && x_stride % 8 == 0 && slot_stride % 4 == 0 && state_off % 4 == 0 &&
                         (((uintptr_t)x | (uintptr_t)mu | (uintptr_t)state | (uintptr_t)out) % 16) == 0;
    if (by_four) {
        if (is_bf16)
            token_shift_mix4_kernel<<<tokens, threads, 0, stream>>>((const __nv_bfloat16*)x, x_stride, mu, n_mix, state, (size_t)slot_stride, state_off, slots, token_row,
                                                                    row_start, (__nv_bfloat16*)out, tokens, hidden);
        else
            token_shift_mix4_kernel<<<tokens, threads, 0, stream>>>((const float*)x, x_stride, mu, n_mix, state, (size_t)slot_stride, state_off, slots, token_row, row_start,
                                                                    (float*)out, tokens, hidden);
        return launch_status();
    }
    if (is_bf16)
        token_shift_mix_kernel<<<tokens, threads, 0, stream>>>((const __nv_bfloat16*)x, x_stride, mu, n_mix, state, (size_t)slot_stride, state_off, slots, token_row,
                                                               row_start, (__nv_bfloat16*)out, tokens, hidden);
    else
        token_shift_mix_kernel<<<tokens, threads, 0, stream>>>((const float*)x, x_stride, mu, n_mix, state, (size_t)slot_stride, state_off, slots, token_row, row_start,
                                                               (float*)out, tokens, hidden);
    return launch_status();
}

HB_EXPORT int hb_token_shift_keep(const void* x, int is_bf16, int x_stride, float* state, long long slot_stride, int state_off, const int* slots,
                                  const int* row_start, int rows, int hidden, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0) return HB_UNSUPPORTED_SIZE;
    if (is_bf16) token_shift_keep_kernel<<<rows, 256, 0, stream>>>((const __nv_bfloat16*)x, x_stride, state, (size_t)slot_stride, state_off, slots, row_start, hidden);
    else token_shift_keep_kernel<<<rows, 256, 0, stream>>>((const float*)x, x_stride, state, (size_t)slot_stride, state_off, slots, row_start, hidden);
    return launch_status();
}

// out[i] = tanh(x[i]) of a dense float tensor, rounded once to the output's type.
HB_EXPORT int hb_tanh_rows(const float* x, void* out, int out_is_bf16, long long count, cudaStream_t stream) {
    if (count <= 0) return 0;
    const long long wanted = (count + 255) / 256;
    const int blocks = (int)(wanted < 2048 ? wanted : 2048);
    if (out_is_bf16) tanh_rows_kernel<<<blocks, 256, 0, stream>>>(x, (__nv_bfloat16*)out, count);
    else tanh_rows_kernel<<<blocks, 256, 0, stream>>>(x, (float*)out, count);
    return launch_status();
}

HB_EXPORT int hb_gated_group_norm(const float* y, int y_stride, const float* gate, int gate_stride, int gate_off, const float* weight,
                                  int weight_len, int group, int groups, int gate_first, float eps, float scale, void* out, int out_is_bf16,
                                  int out_stride, int tokens, int sigmoid_gate, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (group <= 0 || groups <= 0 || groups > 65535 || (weight && weight_len <= 0)) return HB_UNSUPPORTED_SIZE;
    if (!weight) weight_len = 1;
    if (group <= 1024) {
        const dim3 warps(tokens, (groups + 3) / 4);
        if (out_is_bf16)
            gated_group_norm_warp_kernel<<<warps, 128, 0, stream>>>(y, y_stride, gate, gate_stride, gate_off, weight, weight_len, group, groups, gate_first,
                                                                    eps, scale, (__nv_bfloat16*)out, out_stride, sigmoid_gate);
        else
            gated_group_norm_warp_kernel<<<warps, 128, 0, stream>>>(y, y_stride, gate, gate_stride, gate_off, weight, weight_len, group, groups, gate_first,
                                                                    eps, scale, (float*)out, out_stride, sigmoid_gate);
        return launch_status();
    }
    const int threads = group >= 4096 ? 1024 : (group >= 2048 ? 512 : 256);  // a wide group (one norm over all heads): fewer trips per thread
    const dim3 grid(tokens, groups);
    if (out_is_bf16)
        gated_group_norm_kernel<<<grid, threads, 0, stream>>>(y, y_stride, gate, gate_stride, gate_off, weight, weight_len, group, gate_first, eps, scale,
                                                              (__nv_bfloat16*)out, out_stride, sigmoid_gate);
    else
        gated_group_norm_kernel<<<grid, threads, 0, stream>>>(y, y_stride, gate, gate_stride, gate_off, weight, weight_len, group, gate_first, eps, scale,
                                                              (float*)out, out_stride, sigmoid_gate);
    return launch_status();
}

// ---------------------------------------------------------------- a convolution added to its own input
// out[t, c] = x[t, c] + sum_j weight[c, j] * x[t - (taps - 1 - j), c] over the tokens of t's own request (the last column of the weight
// multiplies the current token); inputs before the row's first token come from the request's state (its last taps - 1 inputs as floats,
// oldest first; zero for a new request).  Rows and result share an element type; the sum is float, rounded once.
// hb_conv_state_keep then stores every row's last taps - 1 inputs for the next step.  silu_columns: silu in place over some columns of float rows
// (a recurrence whose keys, queries and values are activated projections; taken inside the scan's preparation it cost more than this pass).
namespace {
template <typename T>
__global__ void residual_conv_kernel(const T* __restrict__ x, int x_stride, int channels, const float* __restrict__ weight, int taps,
                                     const float* __restrict__ state, size_t slot_stride, int state_off, const int* __restrict__ slots,
                                     const int* __restrict__ token_row, const int* __restrict__ row_start, T* __restrict__ out, int out_stride, int first_token) {
    const int t = first_token + blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int r = token_row[t];
    const int i = t - row_start[r];
    const float* kept = state + (size_t)slots[r] * slot_stride + state_off;
    float acc = 0.f;
    for (int j = taps - 1; j >= 0; --j) {  // oldest input first
        const float w = weight[(size_t)c * taps + taps - 1 - j];
        const float v = (i - j >= 0) ? to_float(x[(size_t)(t - j) * x_stride + c]) : kept[(size_t)(taps - 1 + i - j) * channels + c];
        acc = fmaf(w, v, acc);
    }
    out[(size_t)t * out_stride + c] = from_float<T>(to_float(x[(size_t)t * x_stride + c]) + acc);
}

// The same for bfloat16 rows that are whole 16-byte pieces: a thread takes eight neighbouring channels of a token; their 8 * TAPS weights lie
// side by side and are read in 16-byte pieces.
template <int TAPS>
__global__ void residual_conv_bf16x8_kernel(const __nv_bfloat16* __restrict__ x, int x_stride, int channels, const float* __restrict__ weight, int taps,
                                            const float* __restrict__ state, size_t slot_stride, int state_off, const int* __restrict__ slots,
                                            const int* __restrict__ token_row, const int* __restrict__ row_start, __nv_bfloat16* __restrict__ out, int out_stride,
                                            int first_token) {
    const int t = first_token + blockIdx.y, c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= channels) return;
    const int r = token_row[t];
    const int i = t - row_start[r];
    const float* kept = state + (size_t)slots[r] * slot_stride + state_off;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, now[8];
    float w[8 * TAPS];
#pragma unroll
    for (int k = 0; k < 2 * TAPS; ++k) {
        const float4 piece = *reinterpret_cast<const float4*>(weight + (size_t)c * TAPS + 4 * k);
        w[4 * k] = piece.x; w[4 * k + 1] = piece.y; w[4 * k + 2] = piece.z; w[4 * k + 3] = piece.w;
    }
#pragma unroll
    for (int j = TAPS - 1; j >= 0; --j) {  // oldest input first
        float v[8];
        if (i - j >= 0) {
            const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)(t - j) * x_stride + c);
            const __nv_bfloat162* in = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int k = 0; k < 4; ++k) { const float2 f = __bfloat1622float2(in[k]); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
        } else {
            const float* p = kept + (size_t)(TAPS - 1 + i - j) * channels + c;
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = p[k];
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            acc[k] = fmaf(w[k * TAPS + TAPS - 1 - j], v[k], acc[k]);
            if (j == 0) now[k] = v[k];
        }
    }
    uint4 packed;
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int k = 0; k < 4; ++k) o[k] = __floats2bfloat162_rn(now[2 * k] + acc[2 * k], now[2 * k + 1] + acc[2 * k + 1]);
    *reinterpret_cast<uint4*>(out + (size_t)t * out_stride + c) = packed;
}

__global__ void silu_columns_kernel(float* __restrict__ x, int x_stride, int col0, int columns, long long count) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
        float* p = x + (size_t)(i / columns) * x_stride + col0 + (int)(i % columns);
        *p = silu_f(*p);
    }
}

template <typename T>
__global__ void conv_state_keep_kernel(const T* __restrict__ x, int x_stride, int channels, int taps, float* __restrict__ state, size_t slot_stride,
                                       int state_off, const int* __restrict__ slots, const int* __restrict__ row_start, int rows) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
    if (c >= channels || r >= rows) return;
    const int first = row_start[r], n = row_start[r + 1] - first, keep = taps - 1;
    float* kept = state + (size_t)slots[r] * slot_stride + state_off;
    for (int s = 0; s < keep; ++s) {  // ascending: an old entry is read (at s + n > s) before it is overwritten
        const int src = n - keep + s;
        kept[(size_t)s * channels + c] = src >= 0 ? to_float(x[(size_t)(first + src) * x_stride + c]) : kept[(size_t)(s + n) * channels + c];
    }
}
}  // namespace

HB_EXPORT int hb_residual_conv(const void* x, int is_bf16, int x_stride, int channels, const float* weight, int taps, const float* state,
                               long long slot_stride, int state_off, const int* slots, const int* token_row, const int* row_start, void* out,
                               int out_stride, int tokens, cudaStream_t stream) {
    if (tokens <= 0 || channels <= 0) return 0;
    if (taps < 1) return HB_BAD_ARGUMENT;
    const bool by_eight = is_bf16 && taps <= 8 && channels % 8 == 0 && x_stride % 8 == 0 && out_stride % 8 == 0 &&
                          (((uintptr_t)x | (uintptr_t)out | (uintptr_t)weight) & 15) == 0;
    for (int first = 0; first < tokens; first += 65535) {
        const int count = tokens - first < 65535 ? tokens - first : 65535;
        if (by_eight) {
            const dim3 eights((channels / 8 + 127) / 128, count);
#define HB_CONV8(T)                                                                                                                                       \
    case T:                                                                                                                                               \
        residual_conv_bf16x8_kernel<T><<<eights, 128, 0, stream>>>((const __nv_bfloat16*)x, x_stride, channels, weight, taps, state, (size_t)slot_stride, \
                                                                   state_off, slots, token_row, row_start, (__nv_bfloat16*)out, out_stride, first);      \
        break
            switch (taps) { HB_CONV8(1); HB_CONV8(2); HB_CONV8(3); HB_CONV8(4); HB_CONV8(5); HB_CONV8(6); HB_CONV8(7); HB_CONV8(8); }
#undef HB_CONV8
            continue;
        }
        const dim3 grid((channels + 255) / 256, count);
        if (is_bf16)
            residual_conv_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, x_stride, channels, weight, taps, state, (size_t)slot_stride, state_off, slots,
                                                           token_row, row_start, (__nv_bfloat16*)out, out_stride, first);
        else
            residual_conv_kernel<<<grid, 256, 0, stream>>>((const float*)x, x_stride, channels, weight, taps, state, (size_t)slot_stride, state_off, slots,
                                                           token_row, row_start, (float*)out, out_stride, first);
    }
    return launch_status();
}

HB_EXPORT int hb_silu_columns(float* x, int x_stride, int col0, int columns, int tokens, cudaStream_t stream) {
    if (tokens <= 0 || columns <= 0) return 0;
    const long long count = (long long)tokens * columns, wanted = (count + 255) / 256;
    silu_columns_kernel<<<(int)(wanted < 4096 ? wanted : 4096), 256, 0, stream>>>(x, x_stride, col0, columns, count);
    return launch_status();
}

HB_EXPORT int hb_conv_state_keep(const void* x, int is_bf16, int x_stride, int channels, int taps, float* state, long long slot_stride, int state_off,
                                 const int* slots, const int* row_start, int rows, cudaStream_t stream) {
    if (rows <= 0 || channels <= 0 || taps <= 1) return 0;
    if (rows > 65535) return HB_UNSUPPORTED_SIZE;
    const dim3 grid((channels + 127) / 128, rows);
    if (is_bf16) conv_state_keep_kernel<<<grid, 128, 0, stream>>>((const __nv_bfloat16*)x, x_stride, channels, taps, state, (size_t)slot_stride, state_off, slots, row_start, rows);
    else conv_state_keep_kernel<<<grid, 128, 0, stream>>>((const float*)x, x_stride, channels, taps, state, (size_t)slot_stride, state_off, slots, row_start, rows);
    return launch_status();
}

// ---------------------------------------------------------------- the selective scan (a decay per channel and state entry)
// Per channel c with a state vector S[c, :] of n entries and per token, with a step dt_c = softplus(step input), the channel's
// input x_c, and two vectors B and C (n entries each) that all channels share:
//     S[c, i] <- exp(dt_c A[c, i]) S[c, i] + dt_c x_c B_i;     y_c = (sum_i S[c, i] C_i + D_c x_c) * silu(z_c)
// Channels never meet, so a block of 128 threads walks 32 channels through the tokens of one request's row: four lanes share a
// channel, each holding n / 4 of its entries in registers (groups of four consecutive entries).  The only chain from token to
// token is one multiply-add per entry; steps, exponentials and the products with B wait for nothing.  Tokens pass through
// shared memory in chunks that are fetched while the chunk before is walked.  Sums over n are taken in a fixed order (per lane in
// four chains, then a butterfly over the four lanes).
namespace {
struct SelectiveArgs {
    const float* x;      // [tokens, x_stride]: the channels' inputs (after the convolution and its activation)
    int x_stride;
    const float* dt;     // [tokens, dt_stride]: step inputs per channel (softplus is taken here)
    int dt_stride;
    const float* bc;     // [tokens, bc_stride]: B at b_off, C at c_off
    int bc_stride, b_off, c_off;
    const float* a;      // [inner, n]: A, negative
    const float* skip;   // [inner]: D
    const float* gate;   // [tokens, gate_stride]: z at gate_off
    int gate_stride, gate_off;
    float* state;
    size_t slot_stride;
    int state_off;
    const int* slots;
    const int* row_start;
    void* out;           // [tokens, out_stride], or null: only the states are wanted
    int out_stride;
    int inner, n, n_padded;
    float* dt_sums;      // [rows, inner] or null: the sum of a row's steps per channel (what joins segments scanned side by side)
};

// PRECISE (the float32 mode): a token's update and its output sum are taken in double precision and rounded to float once, the state
// staying a float from token to token.  In float arithmetic the decay exp(dt A), the product dt x B and the update each round, and over
// a thousand tokens of slowly fading state that showed in a deep model's logits (a fourfold error against the same model in double).
template <int NG, typename TO, bool PRECISE>
__global__ void __launch_bounds__(128) selective_scan_kernel(const SelectiveArgs a) {
    constexpr int LPC = 4, CH = 128 / LPC, NP = NG * 4 * LPC, CT = NP >= 128 ? 4 : 16;
    constexpr int NB = CT * NP / 128, NC = CT * CH / 128;
    __shared__ __align__(16) float sb[2][CT][NP];
    __shared__ __align__(16) float sc[2][CT][NP];
    __shared__ float sdt[2][CT][CH], sx[2][CT][CH], sz[2][CT][CH];

    const int row = blockIdx.y, tid = threadIdx.x;
    const int l = tid % LPC, cw = tid / LPC, channel = blockIdx.x * CH + cw;
    const bool owns = channel < a.inner;
    const int t0 = a.row_start[row], t1 = a.row_start[row + 1];
    float* const kept = a.state + (size_t)a.slots[row] * a.slot_stride + a.state_off + (size_t)channel * a.n_padded;

    float s[NG][4], rate[NG][4];
#pragma unroll
    for (int r = 0; r < NG; ++r) {
        const int base = 4 * (LPC * r + l);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (owns && base < a.n_padded) v = *reinterpret_cast<const float4*>(kept + base);
        s[r][0] = v.x; s[r][1] = v.y; s[r][2] = v.z; s[r][3] = v.w;
#pragma unroll
        for (int i = 0; i < 4; ++i) rate[r][i] = (owns && base + i < a.n) ? a.a[(size_t)channel * a.n + base + i] : 0.f;
    }
    const float skip = owns ? a.skip[channel] : 0.f;

    float pb[NB], pc[NB], pdt[NC], px[NC], pz[NC];
    auto prefetch = [&](int first) {
#pragma unroll
        for (int i = 0; i < NB; ++i) {
            const int flat = tid + 128 * i, j = flat / NP, index = flat - j * NP, t = first + j;
            const bool live = t < t1 && index < a.n;
            const float* p = a.bc + (size_t)(live ? t : t0) * a.bc_stride;
            pb[i] = live ? p[a.b_off + index] : 0.f;
            pc[i] = live ? p[a.c_off + index] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < NC; ++i) {
            const int flat = tid + 128 * i, j = flat / CH, c = blockIdx.x * CH + (flat - j * CH), t = first + j;
            const bool live = t < t1 && c < a.inner;
            pdt[i] = live ? a.dt[(size_t)t * a.dt_stride + c] : 0.f;
            px[i] = live ? a.x[(size_t)t * a.x_stride + c] : 0.f;
            pz[i] = live ? a.gate[(size_t)t * a.gate_stride + a.gate_off + c] : 0.f;
        }
    };
    auto publish = [&](int buffer) {
#pragma unroll
        for (int i = 0; i < NB; ++i) {
            const int flat = tid + 128 * i, j = flat / NP, index = flat - j * NP;
            sb[buffer][j][index] = pb[i];
            sc[buffer][j][index] = pc[i];
        }
#pragma unroll
        for (int i = 0; i < NC; ++i) {
            const int flat = tid + 128 * i, j = flat / CH, c = flat - j * CH;
            sdt[buffer][j][c] = softplus_f(pdt[i]);
            sx[buffer][j][c] = px[i];
            sz[buffer][j][c] = silu_f(pz[i]);
        }
    };

    float dt_total = 0.f;
    prefetch(t0);
    publish(0);
    __syncthreads();
    int buffer = 0;
    for (int first = t0; first < t1; first += CT, buffer ^= 1) {
        const bool more = first + CT < t1;
        if (more) prefetch(first + CT);  // in flight while this chunk is walked
        const int count = min(CT, t1 - first);
        for (int j = 0; j < count; ++j) {
            const float dt = sdt[buffer][j][cw], xv = sx[buffer][j][cw];
            const float dx = dt * xv;
            dt_total += dt;
            float part[4] = {0.f, 0.f, 0.f, 0.f};
            double wide[4] = {0., 0., 0., 0.};
#pragma unroll
            for (int r = 0; r < NG; ++r) {
                const float4 b4 = *reinterpret_cast<const float4*>(&sb[buffer][j][4 * (LPC * r + l)]);
                const float4 c4 = *reinterpret_cast<const float4*>(&sc[buffer][j][4 * (LPC * r + l)]);
                const float bv[4] = {b4.x, b4.y, b4.z, b4.w}, cv[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if constexpr (PRECISE) {
                        s[r][i] = (float)fma(exp((double)dt * (double)rate[r][i]), (double)s[r][i], (double)dt * (double)xv * (double)bv[i]);
                        wide[i] = fma((double)s[r][i], (double)cv[i], wide[i]);
                    } else {
                        s[r][i] = fmaf(expf(dt * rate[r][i]), s[r][i], dx * bv[i]);
                        part[i] = fmaf(s[r][i], cv[i], part[i]);
                    }
                }
            }
            float y = PRECISE ? (float)((wide[0] + wide[1]) + (wide[2] + wide[3])) : (part[0] + part[1]) + (part[2] + part[3]);
#pragma unroll
            for (int offset = 1; offset < LPC; offset <<= 1) y += __shfl_xor_sync(0xffffffffu, y, offset);
            if (l == 0 && owns && a.out) {
                const float result = fmaf(skip, xv, y) * sz[buffer][j][cw];
                reinterpret_cast<TO*>(a.out)[(size_t)(first + j) * a.out_stride + channel] = from_float<TO>(result);
            }
        }
        if (!more) break;
        publish(buffer ^ 1);
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < NG; ++r) {
        const int base = 4 * (LPC * r + l);
        if (owns && base < a.n_padded) *reinterpret_cast<float4*>(kept + base) = make_float4(s[r][0], s[r][1], s[r][2], s[r][3]);
    }
    if (a.dt_sums && l == 0 && owns) a.dt_sums[(size_t)row * a.inner + channel] = dt_total;
}

template <typename TO, bool PRECISE>
int launch_selective(const SelectiveArgs& a, int rows, cudaStream_t stream) {
    const int per_lane = (a.n_padded + 15) / 16;  // groups of four entries per lane, four lanes per channel
    const dim3 grid((a.inner + 31) / 32, rows);
    if (per_lane <= 1) selective_scan_kernel<1, TO, PRECISE><<<grid, 128, 0, stream>>>(a);
    else if (per_lane <= 2) selective_scan_kernel<2, TO, PRECISE><<<grid, 128, 0, stream>>>(a);
    else if (per_lane <= 4) selective_scan_kernel<4, TO, PRECISE><<<grid, 128, 0, stream>>>(a);
    else if (per_lane <= 8) selective_scan_kernel<8, TO, PRECISE><<<grid, 128, 0, stream>>>(a);
    else selective_scan_kernel<16, TO, PRECISE><<<grid, 128, 0, stream>>>(a);
    return launch_status();
}
}  // namespace

// The state of (slot, channel) is S[channel, :] in n_padded floats at state + slot * slot_stride + state_off + channel * n_padded; n_padded,
// state_off and slot_stride are multiples of 4.  `a` holds A itself (negative), not its logarithm.  precise: a token's arithmetic in double
// precision, rounded to float once (the float32 mode).
HB_EXPORT int hb_selective_scan(const float* x, int x_stride, const float* dt, int dt_stride, const float* bc, int bc_stride, int b_off, int c_off,
                                const float* a, const float* skip, const float* gate, int gate_stride, int gate_off, float* state,
                                long long slot_stride, int state_off, const int* slots, const int* row_start, void* out, int out_is_bf16,
                                int out_stride, int rows, int inner, int n, int n_padded, float* dt_sums, int precise, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (n <= 0 || n > 256 || inner <= 0 || rows > 65535) return HB_UNSUPPORTED_SIZE;
    if (n_padded < n || (n_padded & 3) || (state_off & 3) || (slot_stride & 3) || (((uintptr_t)state) & 15)) return HB_BAD_ARGUMENT;
    const SelectiveArgs args{x, x_stride, dt, dt_stride, bc, bc_stride, b_off, c_off, a, skip, gate, gate_stride, gate_off, state, (size_t)slot_stride,
                             state_off, slots, row_start, out, out_stride, inner, n, n_padded, dt_sums};
    if (precise) return out_is_bf16 ? launch_selective<__nv_bfloat16, true>(args, rows, stream) : launch_selective<float, true>(args, rows, stream);
    return out_is_bf16 ? launch_selective<__nv_bfloat16, false>(args, rows, stream) : launch_selective<float, false>(args, rows, stream);
}


// ---------------------------------------------------------------- joining the segments of a row that were scanned side by side
// A recurrence that is linear in its state, S <- a S + (something that does not depend on S), can be walked in segments that do not
// wait for one another: every segment is first scanned from a zero state, which gives what it adds (its end state E_j); with the
// segment's total decay A_j the state at the start of segment j + 1 is S_{j+1} = A_j S_j + E_j, a short loop per state entry; then
// every segment is scanned again from its true start.  This kernel is the loop, for a constant decay per head (A_j = decay^length):
// ends[j] holds E_j on entry and S_j on return, and the row's state record ends up holding the state after its last segment.
// The result differs from the one-pass scan by rounding only; it is used where bits need not repeat across cuts of the work.
namespace {
__global__ void join_segments_kernel(float* __restrict__ ends, size_t end_stride, float* __restrict__ state, size_t slot_stride, int state_off,
                                     const int* __restrict__ slots, const int* __restrict__ seg_start, const int* __restrict__ seg_row, int segments,
                                     const float* __restrict__ decay, int per_head, int entries) {
    const int entry = blockIdx.x * blockDim.x + threadIdx.x;
    if (entry >= entries) return;
    const float log_decay = log2f(decay[entry / per_head]);
    constexpr int AHEAD = 8;  // what the segments add is asked for before the chain through them starts: one trip to memory, not one per segment
    int j = 0;
    while (j < segments) {
        const int row = seg_row[j];
        float* kept = state + (size_t)slots[row] * slot_stride + state_off + entry;
        float s = *kept;
        while (j < segments && seg_row[j] == row) {
            float added[AHEAD], fade[AHEAD];
            int count = 0;
#pragma unroll
            for (int k = 0; k < AHEAD; ++k) {
                if (j + k < segments && seg_row[j + k] == row) {
                    added[k] = ends[(size_t)(j + k) * end_stride + entry];
                    const int length = seg_start[j + k + 1] - seg_start[j + k];
                    fade[k] = log_decay == 0.f ? 1.f : exp2f((float)length * log_decay);
                    count = k + 1;
                }
            }
#pragma unroll
            for (int k = 0; k < AHEAD; ++k) {
                if (k < count) {
                    ends[(size_t)(j + k) * end_stride + entry] = s;
                    s = fmaf(fade[k], s, added[k]);
                }
            }
            j += count;
        }
        *kept = s;
    }
}
}  // namespace

// ends [segments, end_stride] float: entry e of segment j at ends[j * end_stride + e], e < entries = heads * per_head; the state of
// row r at state + slots[r] * slot_stride + state_off.  Segments of one row follow one another; seg_start has segments + 1 entries.
HB_EXPORT int hb_join_segments(float* ends, long long end_stride, float* state, long long slot_stride, int state_off, const int* slots,
                               const int* seg_start, const int* seg_row, int segments, const float* decay, int heads, int per_head,
                               cudaStream_t stream) {
    if (segments <= 0) return 0;
    if (heads <= 0 || per_head <= 0) return HB_BAD_ARGUMENT;
    const int entries = heads * per_head;
    join_segments_kernel<<<(entries + 255) / 256, 256, 0, stream>>>(ends, (size_t)end_stride, state, (size_t)slot_stride, state_off, slots, seg_start, seg_row,
                                                                 segments, decay, per_head, entries);
    return launch_status();
}


// The same joining for the selective scan, whose decay differs per channel and state entry: over a segment it is exp(A[c, i] * the sum
// of the channel's steps), which the first pass leaves in dt_sums [segments, inner].
namespace {
__global__ void join_selective_segments_kernel(float* __restrict__ ends, size_t end_stride, float* __restrict__ state, size_t slot_stride, int state_off,
                                               const int* __restrict__ slots, const int* __restrict__ seg_row, int segments, const float* __restrict__ a,
                                               const float* __restrict__ dt_sums, int inner, int n, int n_padded) {
    const int entry = blockIdx.x * blockDim.x + threadIdx.x;
    if (entry >= inner * n_padded) return;
    const int channel = entry / n_padded, i = entry - channel * n_padded;
    const float rate = i < n ? a[(size_t)channel * n + i] : 0.f;
    constexpr int AHEAD = 8;
    int j = 0;
    while (j < segments) {
        const int row = seg_row[j];
        float* kept = state + (size_t)slots[row] * slot_stride + state_off + entry;
        float s = *kept;
        while (j < segments && seg_row[j] == row) {
            float added[AHEAD], fade[AHEAD];
            int count = 0;
#pragma unroll
            for (int k = 0; k < AHEAD; ++k) {
                if (j + k < segments && seg_row[j + k] == row) {
                    added[k] = ends[(size_t)(j + k) * end_stride + entry];
                    fade[k] = expf(rate * dt_sums[(size_t)(j + k) * inner + channel]);
                    count = k + 1;
                }
            }
#pragma unroll
            for (int k = 0; k < AHEAD; ++k) {
                if (k < count) {
                    ends[(size_t)(j + k) * end_stride + entry] = s;
                    s = fmaf(fade[k], s, added[k]);
                }
            }
            j += count;
        }
        *kept = s;
    }
}
}  // namespace

HB_EXPORT int hb_join_selective_segments(float* ends, long long end_stride, float* state, long long slot_stride, int state_off, const int* slots,
                                         const int* seg_row, int segments, const float* a, const float* dt_sums, int inner, int n, int n_padded,
                                         cudaStream_t stream) {
    if (segments <= 0) return 0;
    if (inner <= 0 || n <= 0 || n_padded < n) return HB_BAD_ARGUMENT;
    const int entries = inner * n_padded;
    join_selective_segments_kernel<<<(entries + 255) / 256, 256, 0, stream>>>(ends, (size_t)end_stride, state, (size_t)slot_stride, state_off, slots, seg_row,
                                                                           segments, a, dt_sums, inner, n, n_padded);
    return launch_status();
}
