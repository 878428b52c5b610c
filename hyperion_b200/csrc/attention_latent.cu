// Causal attention of many query heads over ONE shared key/value head whose keys are the cached records of RECORD entries
// and whose values are the records' first VALUE entries (attention over a latent, the up-projections carried to the query and
// output sides).  bfloat16 operands on the tensor cores (mma.sync m16n8k16, float accumulators); scores, the running maximum,
// the sums and the optional sink (one more term exp(sink) per head in the denominator, no key, no value) in float.
//
// A block serves 16 or 32 rows, a row being one (token, head) pair of one request of the step: rows are numbered token by token,
// head by head, so a decoded token with 16 heads is one block and a prompt's portion fills blocks densely whatever the number
// of heads.  Keys are walked in tiles of 64 absolute positions, two tiles in flight (cp.async into two shared-memory buffers,
// rows padded by 16 bytes so that ldmatrix meets no bank twice).  Per tile, with 8 warps:
//   1. scores: warp w takes the 16 rows of row tile w % MT and 8 * MT keys, the whole record as the contraction, and leaves its
//      rows' maxima over its keys in shared memory;
//   2. every such warp forms the rows' new running maxima from all groups' maxima, exponentiates its own scores once, adds them
//      to its part of the rows' sums and writes them as bfloat16 weights to shared memory (and one warp the rescale factors);
//   3. weighted values: warp w owns VALUE / 8 columns of all rows' results in registers, reads the weights as A fragments and the
//      same key tile, transposed by ldmatrix, as B fragments.
// With splits > 1 a block walks only its share of the key tiles and leaves an unnormalised result with its maximum and sum in a
// workspace; a second kernel merges the shares.  A row's result depends on the positions of the key tiles only, never on how the
// request was cut into steps or on the rest of the batch.
#include "common.cuh"
#include <type_traits>

#ifndef HB_RECORD
#define HB_RECORD 576
#endif
#ifndef HB_VALUE
#define HB_VALUE 512
#endif

namespace {
constexpr int RECORD = HB_RECORD, VALUE = HB_VALUE;
static_assert(RECORD % 16 == 0 && VALUE % 8 == 0 && VALUE <= RECORD && RECORD <= 640, "record a multiple of 16 up to 640, value a multiple of 8 within it");
constexpr int BN = 64, WARPS = 8, THREADS = WARPS * 32;
constexpr int KSTEPS = RECORD / 16, CHUNKS = RECORD / 8;  // contraction steps of a score; 16-byte pieces of a record
constexpr int ROW = RECORD + 8, PROW = BN + 8;            // shared-memory strides in elements
constexpr int NT = VALUE / 8, NTW = (NT + WARPS - 1) / WARPS;  // column tiles of the result, and those of one warp

struct LatentArgs {
    const __nv_bfloat16* q;  // [tokens, heads, RECORD] with q_stride elements per token
    int q_stride;
    __nv_bfloat16* out;  // [tokens, heads, VALUE] with out_stride elements per token
    int out_stride;
    float* part;  // splits > 1: [tokens * heads, splits, VALUE + 2]
    const __nv_bfloat16* cache;  // [pages, page_size, RECORD]
    const int* block_table;
    int table_width;
    const int* row_start;  // [rows + 1]
    const int* positions;
    const float* sinks;  // [heads] or null
    int heads, page_size, pages, splits;
    float scale_log2;  // scale * log2(e)
    int* status;
};

__device__ __forceinline__ uint32_t shared_address(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void copy16_async(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(shared_address(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void copies_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int MT>
constexpr size_t shared_bytes() {
    return (size_t)(2 * BN * ROW + 16 * MT * ROW + 16 * MT * PROW) * sizeof(__nv_bfloat16) + (size_t)(128 + 32 + 32 + 128) * sizeof(float);
}

template <int MT>
__global__ void __launch_bounds__(THREADS, 1) attention_latent_kernel(const LatentArgs a) {
    constexpr int M = 16 * MT, GROUPS = WARPS / MT, SN = MT;  // rows of the block; key groups of the score phase; key tiles of 8 per warp there
    extern __shared__ __align__(16) unsigned char shared_raw[];
    __nv_bfloat16* kbuf = reinterpret_cast<__nv_bfloat16*>(shared_raw);  // [2][BN][ROW]
    __nv_bfloat16* qs = kbuf + 2 * BN * ROW;                             // [M][ROW]
    __nv_bfloat16* ps = qs + M * ROW;                                    // [M][PROW]
    float* pmax = reinterpret_cast<float*>(ps + M * PROW);               // [GROUPS][M]
    float* alpha = pmax + 128;                                           // [M]
    float* mfin = alpha + 32;                                            // [M]
    float* lsum = mfin + 32;                                             // [GROUPS][M]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int brow = blockIdx.y, split = blockIdx.z;
    const int t0 = a.row_start[brow], count = a.row_start[brow + 1] - t0;
    const int heads = a.heads, total = count * heads;
    const int base_f = (gridDim.x - 1 - blockIdx.x) * M;  // a request's last rows see the most keys: their blocks start first
    if (base_f >= total) return;
    const int pos_first = a.positions[t0];
    const int hi = pos_first + (min(total, base_f + M) - 1) / heads;  // the last position any row of the block sees
    const int n_tiles = hi / BN + 1;
    const int per_split = (n_tiles + a.splits - 1) / a.splits;
    const int tile_lo = split * per_split, tile_hi = min(n_tiles, tile_lo + per_split);
    const int* table = a.block_table + (size_t)brow * a.table_width;
    bool bad_page = false;

    // queries: rows beyond the request's last are zeros
    for (int idx = tid; idx < M * CHUNKS; idx += THREADS) {
        const int r = idx / CHUNKS, c = idx - r * CHUNKS, f = base_f + r;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (f < total) {
            const int tok = f / heads, head = f - tok * heads;
            v = *reinterpret_cast<const uint4*>(a.q + (size_t)(t0 + tok) * a.q_stride + (size_t)head * RECORD + c * 8);
        }
        *reinterpret_cast<uint4*>(qs + r * ROW + c * 8) = v;
    }

    auto load_tile = [&](int tile, int buf) {  // a warp per key; keys past the block's last position are zeros
        __nv_bfloat16* dst0 = kbuf + (size_t)buf * BN * ROW;
        // lane i looks up the page of the warp's i-th key, so the warp waits for one round of table reads, not for eight in a row
        long long mine = -1;
        if (lane < BN / WARPS) {
            const int j = tile * BN + warp + lane * WARPS;
            if (j <= hi) {
                const int block = j / a.page_size;
                const int page = block < a.table_width ? table[block] : -1;
                if (page < 0 || page >= a.pages) bad_page = true;
                else mine = ((long long)page * a.page_size + (j - block * a.page_size)) * RECORD;
            }
        }
#pragma unroll
        for (int i = 0; i < BN / WARPS; ++i) {
            const long long offset = __shfl_sync(0xffffffffu, mine, i);
            __nv_bfloat16* dst = dst0 + (warp + i * WARPS) * ROW;
            if (offset >= 0) {
                const __nv_bfloat16* src = a.cache + offset;
                for (int c = lane; c < CHUNKS; c += 32) copy16_async(dst + c * 8, src + c * 8);
            } else {
                for (int c = lane; c < CHUNKS; c += 32) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0, 0, 0, 0);
            }
        }
    };

    // the score phase's rows of this thread: g and g + 8 of row tile mt
    const int mt = warp % MT, kg = warp / MT, key0 = kg * 8 * SN;
    int row_pos[2];
    float m_run[2], l_part[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int f = base_f + mt * 16 + g + 8 * h;
        const bool valid = f < total;
        row_pos[h] = valid ? pos_first + f / heads : hi;
        const bool sunk = a.sinks && split == 0;
        m_run[h] = sunk ? a.sinks[min(f, total - 1) % heads] * 1.4426950408889634f : -INFINITY;
        l_part[h] = (sunk && kg == 0 && t == 0) ? 1.f : 0.f;
    }
    float acc[MT][NTW][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int n = 0; n < NTW; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][n][e] = 0.f;
    const int n_first = warp * NTW, n_here = min(NTW, NT - n_first);  // this warp's column tiles of the result (may be none)

    if (tile_lo < tile_hi) load_tile(tile_lo, 0);
    copies_commit();
    const uint32_t q_addr = shared_address(qs + (mt * 16 + (lane & 15)) * ROW + (lane >> 4) * 8);
    const uint32_t p_addr = shared_address(ps + (lane & 15) * PROW + (lane >> 4) * 8);

    for (int tile = tile_lo; tile < tile_hi; ++tile) {
        const int buf = (tile - tile_lo) & 1;
        copies_wait_all();
        __syncthreads();  // the tile is in shared memory, and every warp is done with the tile before it
        if (tile + 1 < tile_hi) load_tile(tile + 1, buf ^ 1);
        copies_commit();
        const __nv_bfloat16* kb = kbuf + (size_t)buf * BN * ROW;

        // 1. scores of 16 rows against 8 * SN keys: fragments are fetched ahead of the products that use them, and four sets of accumulators
        // keep that many chains of products in flight
        constexpr int U = 4;
        float s[U][SN][4];
#pragma unroll
        for (int c = 0; c < U; ++c)
#pragma unroll
            for (int n = 0; n < SN; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[c][n][e] = 0.f;
        const uint32_t k_addr = shared_address(kb + (key0 + ((SN == 2) ? ((lane >> 4) << 3) : 0) + (lane & 7)) * ROW + ((lane >> 3) & 1) * 8);
        constexpr int AHEAD = 3;  // a step's fragments are asked for three steps before its products are issued
        uint32_t qa[AHEAD + 1][4], kf[AHEAD + 1][4];
#pragma unroll
        for (int ks = 0; ks < KSTEPS + AHEAD; ++ks) {
            if (ks < KSTEPS) {
                ldmatrix_x4(qa[ks % (AHEAD + 1)], q_addr + ks * 32);
                if constexpr (SN == 2) {
                    ldmatrix_x4(kf[ks % (AHEAD + 1)], k_addr + ks * 32);
                } else {
                    uint32_t two[2];
                    ldmatrix_x2(two, k_addr + ks * 32);
                    kf[ks % (AHEAD + 1)][0] = two[0], kf[ks % (AHEAD + 1)][1] = two[1];
                }
            }
            if (ks >= AHEAD) {
                const int at = ks - AHEAD;
                mma_bf16(s[at % U][0], qa[at % (AHEAD + 1)], kf[at % (AHEAD + 1)][0], kf[at % (AHEAD + 1)][1]);
                if constexpr (SN == 2) mma_bf16(s[at % U][SN - 1], qa[at % (AHEAD + 1)], kf[at % (AHEAD + 1)][2], kf[at % (AHEAD + 1)][3]);
            }
        }
#pragma unroll
        for (int n = 0; n < SN; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[0][n][e] = (s[0][n][e] + s[1][n][e]) + (s[2][n][e] + s[3][n][e]);
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < SN; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = tile * BN + key0 + n * 8 + 2 * t + (e & 1);
                const float v = (j <= row_pos[e >> 1]) ? s[0][n][e] * a.scale_log2 : -INFINITY;
                s[0][n][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            if (t == 0) pmax[kg * M + mt * 16 + g + 8 * h] = mx[h];
        }
        __syncthreads();

        // 2. the rows' new maxima, the weights once, the rescale factors
        float m_use[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = mt * 16 + g + 8 * h;
            float m_new = m_run[h];
#pragma unroll
            for (int k = 0; k < GROUPS; ++k) m_new = fmaxf(m_new, pmax[k * M + r]);
            m_use[h] = m_new == -INFINITY ? 0.f : m_new;
            const float al = exp2f(m_run[h] - m_use[h]);
            l_part[h] *= al;
            m_run[h] = m_new;
            if (kg == 0 && t == 0) alpha[r] = al;
        }
#pragma unroll
        for (int n = 0; n < SN; ++n) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float p0 = exp2f(s[0][n][2 * h] - m_use[h]), p1 = exp2f(s[0][n][2 * h + 1] - m_use[h]);
                l_part[h] += p0 + p1;
                *reinterpret_cast<__nv_bfloat162*>(ps + (mt * 16 + g + 8 * h) * PROW + key0 + n * 8 + 2 * t) = __floats2bfloat162_rn(p0, p1);
            }
        }
        __syncthreads();

        // 3. results: rescale, then weights [M, 64] times the records' first VALUE entries [64, this warp's columns]
        if (n_here > 0) {
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                const float a0 = alpha[i * 16 + g], a1 = alpha[i * 16 + g + 8];
#pragma unroll
                for (int n = 0; n < NTW; ++n) {
                    acc[i][n][0] *= a0, acc[i][n][1] *= a0;
                    acc[i][n][2] *= a1, acc[i][n][3] *= a1;
                }
            }
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) {
                uint32_t pa[MT][4];
#pragma unroll
                for (int i = 0; i < MT; ++i) ldmatrix_x4(pa[i], p_addr + (i * 16 * PROW + kk * 16) * 2);
                const __nv_bfloat16* vrow = kb + (kk * 16 + (lane & 15)) * ROW + n_first * 8;
                // all of this step's value fragments first, then its products
                uint32_t vb[(NTW + 1) / 2][4];
#pragma unroll
                for (int n = 0; n < NTW; n += 2) {
                    if (n + 1 < n_here) {
                        ldmatrix_x4_trans(vb[n / 2], shared_address(vrow + n * 8 + (lane >> 4) * 8));
                    } else if (n < n_here) {
                        uint32_t two[2];
                        ldmatrix_x2_trans(two, shared_address(vrow + n * 8));
                        vb[n / 2][0] = two[0], vb[n / 2][1] = two[1];
                    }
                }
#pragma unroll
                for (int n = 0; n < NTW; n += 2) {
                    if (n < n_here) {
#pragma unroll
                        for (int i = 0; i < MT; ++i) mma_bf16(acc[i][n], pa[i], vb[n / 2][0], vb[n / 2][1]);
                    }
                    if (n + 1 < n_here && n + 1 < NTW) {
#pragma unroll
                        for (int i = 0; i < MT; ++i) mma_bf16(acc[i][n + 1 < NTW ? n + 1 : n], pa[i], vb[n / 2][2], vb[n / 2][3]);
                    }
                }
            }
        }
    }
    copies_wait_all();
    if (bad_page) atomicOr(a.status, HB_STATUS_BAD_PAGE);

    // the rows' sums: the parts of the four lanes of a row, then of the key groups
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float l = l_part[h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (t == 0) {
            lsum[kg * M + mt * 16 + g + 8 * h] = l;
            if (kg == 0) mfin[mt * 16 + g + 8 * h] = m_run[h];
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < MT; ++i) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = i * 16 + g + 8 * h, f = base_f + r;
            if (f >= total) continue;
            float l = 0.f;
#pragma unroll
            for (int k = 0; k < GROUPS; ++k) l += lsum[k * M + r];
            const int tok = f / heads, head = f - tok * heads;
            if (a.splits == 1) {
                const float inv = l > 0.f ? 1.f / l : 0.f;
                __nv_bfloat16* dst = a.out + (size_t)(t0 + tok) * a.out_stride + (size_t)head * VALUE;
#pragma unroll
                for (int n = 0; n < NTW; ++n)
                    if (n < n_here)
                        *reinterpret_cast<__nv_bfloat162*>(dst + (n_first + n) * 8 + 2 * t) =
                            __floats2bfloat162_rn(acc[i][n][2 * h] * inv, acc[i][n][2 * h + 1] * inv);
            } else {
                float* dst = a.part + ((size_t)((size_t)t0 * heads + f) * a.splits + split) * (VALUE + 2);
#pragma unroll
                for (int n = 0; n < NTW; ++n)
                    if (n < n_here) *reinterpret_cast<float2*>(dst + (n_first + n) * 8 + 2 * t) = make_float2(acc[i][n][2 * h], acc[i][n][2 * h + 1]);
                if (warp == 0 && t == 0) dst[VALUE] = mfin[r], dst[VALUE + 1] = l;
            }
        }
    }
}

// One block per (token, head): the shares of the key splits, each with its maximum and sum, become one normalised result.
__global__ void __launch_bounds__(128) attention_latent_merge_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out, int out_stride, int heads,
                                                                      int splits) {
    const int f = blockIdx.x, tok = f / heads, head = f - tok * heads;
    const float* mine = part + (size_t)f * splits * (VALUE + 2);
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, mine[(size_t)s * (VALUE + 2) + VALUE]);
    const float m_use = m == -INFINITY ? 0.f : m;
    float l = 0.f;
    for (int s = 0; s < splits; ++s) l += mine[(size_t)s * (VALUE + 2) + VALUE + 1] * exp2f(mine[(size_t)s * (VALUE + 2) + VALUE] - m_use);
    const float inv = l > 0.f ? 1.f / l : 0.f;
    for (int d = threadIdx.x; d < VALUE; d += 128) {
        float sum = 0.f;
        for (int s = 0; s < splits; ++s) sum += mine[(size_t)s * (VALUE + 2) + d] * exp2f(mine[(size_t)s * (VALUE + 2) + VALUE] - m_use);
        out[(size_t)tok * out_stride + (size_t)head * VALUE + d] = __float2bfloat16_rn(sum * inv);
    }
}

template <int MT>
int launch_latent(const LatentArgs& a, int rows, int longest_count, cudaStream_t stream) {
    static bool raised = false;
    const size_t bytes = shared_bytes<MT>();
    if (!raised) {
        const cudaError_t e = cudaFuncSetAttribute(attention_latent_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    const long long per_row = ((long long)longest_count * a.heads + 16 * MT - 1) / (16 * MT);
    if (per_row > 0x7fffffffLL || rows > 65535 || a.splits > 65535) return HB_UNSUPPORTED_SIZE;
    attention_latent_kernel<MT><<<dim3((unsigned)per_row, rows, a.splits), THREADS, bytes, stream>>>(a);
    return launch_status();
}
}  // namespace

HB_EXPORT int hb_attention_latent_sizes(int* record, int* value) {
    *record = RECORD, *value = VALUE;
    return 0;
}

// q [tokens, heads, RECORD] bfloat16 (q_stride elements per token); cache [pages, page_size, RECORD]; out [tokens, heads, VALUE]
// (out_stride per token).  row_start [rows + 1]: the tokens of request row r are row_start[r] .. row_start[r + 1] - 1 at consecutive
// positions; longest_count: the most tokens any row has (it sizes the grid).  wide_rows: blocks of 32 rows instead of 16.
// splits > 1: every block walks one share of its key tiles and `part` holds tokens * heads * splits * (VALUE + 2) floats.
HB_EXPORT int hb_attention_latent(const void* q, int q_stride, void* out, int out_stride, float* part, const void* cache, const int* block_table,
                                  int table_width, const int* row_start, const int* positions, const float* sinks, int tokens, int rows,
                                  int longest_count, int heads, int page_size, int pages, int splits, int wide_rows, float scale, int* status,
                                  cudaStream_t stream) {
    if (tokens <= 0 || rows <= 0) return 0;
    if (heads <= 0 || page_size <= 0 || splits <= 0 || longest_count <= 0 || (splits > 1 && !part)) return HB_BAD_ARGUMENT;
    if ((q_stride % 8) || (out_stride % 2) || ((uintptr_t)q % 16) || ((uintptr_t)cache % 16) || ((uintptr_t)out % 4)) return HB_BAD_ARGUMENT;
    const LatentArgs a{(const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, part, (const __nv_bfloat16*)cache, block_table, table_width,
                       row_start, positions, sinks, heads, page_size, pages, splits, scale * 1.4426950408889634f, status};
    const int code = wide_rows ? launch_latent<2>(a, rows, longest_count, stream) : launch_latent<1>(a, rows, longest_count, stream);
    if (code || splits == 1) return code;
    attention_latent_merge_kernel<<<tokens * heads, 128, 0, stream>>>(part, (__nv_bfloat16*)out, out_stride, heads, splits);
    return launch_status();
}
