// Causal grouped-query attention WITHOUT a softmax, with the heads' scores mixed before the weights are
// formed. For a query at position p and every key j it sees (j <= p, and p - j < window where there is a
// window):
//
//     s_a  = scale * q_a . k_g(a),j                      for every query head a (g(a): its key/value head)
//     s_a <- sum_b talk[a, b] * s_b                      (optional: a matrix over the heads)
//     w_a  = sigmoid(s_a + head_bias[a])                 (optional bias; no normalisation over the keys)
//     o_a  = out_scale * sum_j w_a,j * v_g(a),j
//
// Because the mix needs the scores of ALL heads for one (query, key) pair, a key is handled for all heads at
// once. Scores, the mix, the weights and the sums are 32-bit.
//
// sigmoid_attention_generic: one block per (token, head a), four warps; the queries of all heads lie in
// shared memory; warp w takes the visible keys first + w, first + w + 4, ...; for a key it forms the scores
// of all heads (lanes over the head's elements), mixes row a of the matrix, and adds w_a * v to its partial
// sum; the four partial sums are added in a fixed order. Which keys a query sees and the order in which they
// are reduced depend only on its position and the window, so a token's result does not depend on the batch
// or on how the tokens were cut into steps. Any head and value size up to 256, any group; both dtypes.
//
// sigmoid_attention_tiles (bfloat16, the head and value sizes of LLMB_SIGMOID_SHAPES): tiles of 64 queries
// of one head on mma.sync, over the pages the tile's windows reach. The mix is linear in the queries, so it
// is done on them: with G key/value heads, the mixed score of head a is
//     sum over g of (sum over the heads b of group g of talk[a, b] q_b) . k_g,
// one product of a "mixed query" of G * dim elements with the keys of all G heads at a position. A block
// (eight warps: two share 16 query rows and take half of a page's keys each; their sums meet at the end)
// forms its tile's mixed queries once (32-bit sums, rounded to bfloat16 as any query is) in shared memory;
// per page it runs the G key tiles and then the value tile of its own group through a ring of three
// buffers (cp.async, two units in flight), S accumulating over the key tiles in 32-bit; the weights
// sigmoid(scale S + bias) are formed in 32-bit, masked at the diagonal and at the window's lower edge, and
// become the A operand of the second product. Nothing is normalised, so there is no running maximum and no
// rescaling. Without a matrix the mixed query is the head's own and G is 1. The price of mixing is G times
// the score products of a plain attention. Steps in which every sequence brings one token have a kernel of
// their own (below); this one also serves them (one live row a tile) where that one does not.
#include "common.cuh"
#include "mma.cuh"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_sigmoid_attention)

constexpr int MAX_PER_LANE = LLMB_MAX_HEAD_DIM / 32;
constexpr int WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
sigmoid_attention_generic_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                                 const T* __restrict__ v_cache, const int* __restrict__ block_table, int table_stride,
                                 int ring_pages, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                 T* __restrict__ out, int out_stride, int n_heads, int n_kv_heads, int dim, int vdim,
                                 float scale, int window, const float* __restrict__ talk,
                                 const float* __restrict__ head_bias, float out_scale) {
    extern __shared__ float shared[];
    float* q_all = shared;                              // [n_heads * dim]
    float* mix_row = shared + (size_t)n_heads * dim;    // [n_heads]: row `head` of the matrix
    float* partial = mix_row + n_heads;                 // [WARPS][32 * MAX_PER_LANE]
    int t = blockIdx.x, head = blockIdx.y;
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int group = n_heads / n_kv_heads;
    int kv_head = head / group;
    int pos = tok_pos[t];
    int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int* pages = block_table + (size_t)tok_seq[t] * table_stride;
    const T* q_row = q + (size_t)t * q_stride;
    for (int e = threadIdx.x; e < n_heads * dim; e += WARPS * 32) q_all[e] = to_float(q_row[e]);
    for (int e = threadIdx.x; e < n_heads; e += WARPS * 32) mix_row[e] = talk ? talk[(size_t)head * n_heads + e] : (e == head ? 1.f : 0.f);
    __syncthreads();
    float bias = head_bias ? head_bias[head] : 0.f;

    float acc[MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) acc[i] = 0.f;

    for (int j = first + warp; j <= pos; j += WARPS) {
        size_t page = (size_t)pages[(j / LLMB_PAGE) % ring_pages];
        int slot_row = j % LLMB_PAGE;
        float mixed = 0.f;
        // without a matrix only the head's own score is needed: its key/value head alone
        int g_first = talk ? 0 : kv_head, g_last = talk ? n_kv_heads : kv_head + 1;
        for (int g = g_first; g < g_last; ++g) {
            const T* key = k_cache + ((page * n_kv_heads + g) * LLMB_PAGE + slot_row) * dim;
            float kv[MAX_PER_LANE];
#pragma unroll
            for (int i = 0; i < MAX_PER_LANE; ++i) {
                int d = lane + 32 * i;
                kv[i] = d < dim ? to_float(key[d]) : 0.f;
            }
            int a_first = talk ? g * group : head, a_last = talk ? (g + 1) * group : head + 1;
            for (int a = a_first; a < a_last; ++a) {
                const float* qa = q_all + (size_t)a * dim;
                float dot = 0.f;
#pragma unroll
                for (int i = 0; i < MAX_PER_LANE; ++i) {
                    int d = lane + 32 * i;
                    if (d < dim) dot = fmaf(qa[d], kv[i], dot);
                }
                mixed = fmaf(mix_row[a], warp_sum(dot) * scale, mixed);
            }
        }
        float w = 1.0f / (1.0f + expf(-(mixed + bias)));
        const T* value = v_cache + ((page * n_kv_heads + kv_head) * LLMB_PAGE + slot_row) * vdim;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            int d = lane + 32 * i;
            if (d < vdim) acc[i] = fmaf(w, to_float(value[d]), acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) partial[warp * 32 * MAX_PER_LANE + lane + 32 * i] = acc[i];
    __syncthreads();
    if (warp == 0) {
        T* o = out + (size_t)t * out_stride + (size_t)head * vdim;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            int d = lane + 32 * i;
            if (d < vdim) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < WARPS; ++w) v += partial[w * 32 * MAX_PER_LANE + d];
                o[d] = from_float<T>(v * out_scale);
            }
        }
    }
}

LLMB_EXPORT int llmb_sigmoid_attention_generic(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                               const int* block_table, int table_stride, int ring_pages,
                                               const int* tok_pos, const int* tok_seq, void* out, int out_stride,
                                               int dtype, int n_tokens, int n_heads, int n_kv_heads, int dim, int vdim,
                                               float scale, int window, const float* talk, const float* head_bias,
                                               float out_scale, cudaStream_t stream) {
    if (n_tokens == 0) return LLMB_OK;
    LLMB_REQUIRE(dim > 0 && dim <= LLMB_MAX_HEAD_DIM && vdim > 0 && vdim <= LLMB_MAX_HEAD_DIM,
                 "sigmoid_attention_generic: head size %d or value size %d exceeds %d", dim, vdim, LLMB_MAX_HEAD_DIM);
    LLMB_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 && n_heads <= 128,
                 "sigmoid_attention_generic: %d heads are no multiple of %d kv heads (or more than 128)", n_heads,
                 n_kv_heads);
    LLMB_REQUIRE(ring_pages > 0 && window >= 0, "sigmoid_attention_generic: bad sizes");
    size_t smem = sizeof(float) * ((size_t)n_heads * dim + n_heads + (size_t)WARPS * 32 * MAX_PER_LANE);
    LLMB_REQUIRE(smem <= 200 * 1024, "sigmoid_attention_generic: %d heads of %d do not fit in shared memory", n_heads, dim);
    dim3 grid(n_tokens, n_heads);
#define LLMB_SIGMOID(T)                                                                                             \
    do {                                                                                                            \
        if (smem > 48 * 1024)                                                                                       \
            LLMB_CUDA(cudaFuncSetAttribute(sigmoid_attention_generic_kernel<T>,                                     \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                \
        sigmoid_attention_generic_kernel<T><<<grid, WARPS * 32, smem, stream>>>(                                    \
            (const T*)q, q_stride, (const T*)k_cache, (const T*)v_cache, block_table, table_stride, ring_pages,     \
            tok_pos, tok_seq, (T*)out, out_stride, n_heads, n_kv_heads, dim, vdim, scale, window, talk, head_bias,  \
            out_scale);                                                                                             \
    } while (0)
    if (dtype == LLMB_DTYPE_F32) LLMB_SIGMOID(float);
    else if (dtype == LLMB_DTYPE_BF16) LLMB_SIGMOID(__nv_bfloat16);
    else return fail(LLMB_ERR_ARGUMENT, "sigmoid_attention_generic: unknown dtype %d", dtype);
#undef LLMB_SIGMOID
    return check_launch("sigmoid_attention_generic");
}

// ----------------------------------------------------------------------------- tiles on the tensor cores

constexpr int BQ = WARPS * 16;               // queries per block
constexpr int TILE_WARPS = 2 * WARPS;        // two warps share 16 query rows and halve a page's keys
constexpr int STAGES = 3;
constexpr int PAD = 8;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D, int DV>
__global__ void __launch_bounds__(TILE_WARPS * 32)
sigmoid_attention_tiles_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ k_cache,
                               const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table,
                               int table_stride, int ring_pages, const int* __restrict__ cu_seqlens,
                               const int* __restrict__ seq_lens, __nv_bfloat16* __restrict__ out, int out_stride,
                               int n_heads, int n_kv_heads, float scale, int window, const float* __restrict__ talk,
                               const float* __restrict__ head_bias, float out_scale) {
    constexpr int LDS = (D > DV ? D : DV) + PAD;
    constexpr int TILE_ELEMS = LLMB_PAGE * LDS;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    int seq = blockIdx.z, head = blockIdx.x;
    int first_token = cu_seqlens[seq];
    int n_new = cu_seqlens[seq + 1] - first_token;
    int n_tiles = (n_new + BQ - 1) / BQ;
    if ((int)blockIdx.y >= n_tiles) return;
    int tile = n_tiles - 1 - blockIdx.y;
    int start = seq_lens[seq] - n_new;
    int group = n_heads / n_kv_heads;
    int kv_head = head / group;
    int g_first = talk ? 0 : kv_head, g_count = talk ? n_kv_heads : 1;     // the key heads whose scores enter
    int ldq = g_count * D + PAD;
    __nv_bfloat16* mixed = reinterpret_cast<__nv_bfloat16*>(smem_raw);     // [BQ][ldq]
    __nv_bfloat16* ring = mixed + (size_t)BQ * ldq;                         // [STAGES][64][LDS]
    // eight warps: warps w and w + 4 share the 16 query rows of w and take the first and the second 32 keys of a page
    int tid = threadIdx.x, warp = (tid >> 5) & 3, half = tid >> 7, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int* pages = block_table + (size_t)seq * table_stride;

    int row0 = tile * BQ + warp * 16 + g, row1 = row0 + 8;
    int pos0 = start + row0, pos1 = start + row1;
    int warp_last_pos = start + min(tile * BQ + warp * 16 + 15, n_new - 1);
    if (tile * BQ + warp * 16 >= n_new) warp_last_pos = -1;
    int tile_last_pos = start + min(tile * BQ + BQ - 1, n_new - 1);
    int n_pages = tile_last_pos / LLMB_PAGE + 1;
    int tile_oldest = window > 0 ? max(start + tile * BQ - window + 1, 0) : 0;
    int first_page = tile_oldest / LLMB_PAGE;
    int warp_oldest = window > 0 ? max(start + tile * BQ + warp * 16 - window + 1, 0) : 0;
    int low0 = window > 0 ? pos0 - window + 1 : 0, low1 = window > 0 ? pos1 - window + 1 : 0;

    int units_per_page = g_count + 1;
    int n_units = (n_pages - first_page) * units_per_page;
    auto load_unit = [&](int n) {
        int p = first_page + n / units_per_page, i = n % units_per_page;
        size_t page = (size_t)pages[p % ring_pages];
        __nv_bfloat16* to = ring + (size_t)(n % STAGES) * TILE_ELEMS;
        if (i < g_count) {
            const __nv_bfloat16* from = k_cache + ((page * n_kv_heads + g_first + i) * LLMB_PAGE) * D;
            for (int c = tid; c < LLMB_PAGE * (D / 8); c += TILE_WARPS * 32) {
                int row = c / (D / 8), col = (c % (D / 8)) * 8;
                cp_async16(to + row * LDS + col, from + (size_t)row * D + col);
            }
        } else {
            const __nv_bfloat16* from = v_cache + ((page * n_kv_heads + kv_head) * LLMB_PAGE) * DV;
            for (int c = tid; c < LLMB_PAGE * (DV / 8); c += TILE_WARPS * 32) {
                int row = c / (DV / 8), col = (c % (DV / 8)) * 8;
                cp_async16(to + row * LDS + col, from + (size_t)row * DV + col);
            }
        }
    };
    if (n_units > 0) load_unit(0);
    cp_async_commit();
    if (n_units > 1) load_unit(1);
    cp_async_commit();

    // the tile's mixed queries: for key head g, sum over the heads b of its group of talk[head, b] * q_b
    {
        int pairs = g_count * D / 2;
        for (int idx = tid; idx < BQ * pairs; idx += TILE_WARPS * 32) {
            int r = idx / pairs, c = (idx % pairs) * 2;
            int gi = c / D, d = c % D;
            int row = tile * BQ + r;
            float lo = 0.f, hi = 0.f;
            if (row < n_new) {
                const __nv_bfloat16* q_row = q + (size_t)(first_token + row) * q_stride;
                if (talk) {
                    for (int b = 0; b < group; ++b) {
                        int other = (g_first + gi) * group + b;
                        float w = talk[(size_t)head * n_heads + other];
                        lo = fmaf(w, to_float(q_row[(size_t)other * D + d]), lo);
                        hi = fmaf(w, to_float(q_row[(size_t)other * D + d + 1]), hi);
                    }
                } else {
                    lo = to_float(q_row[(size_t)head * D + d]);
                    hi = to_float(q_row[(size_t)head * D + d + 1]);
                }
            }
            *reinterpret_cast<__nv_bfloat162*>(mixed + (size_t)r * ldq + c) = __floats2bfloat162_rn(lo, hi);
        }
    }
    float bias = head_bias ? head_bias[head] : 0.f;
    // sigmoid(z) = 1 / (1 + 2^(-z log2 e)), z = scale * s + bias
    float slope = -scale * 1.4426950408889634f, offset = -bias * 1.4426950408889634f;

    float acc[DV / 8][4];
#pragma unroll
    for (int n = 0; n < DV / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
    float s[4][4];

    for (int n = 0; n < n_units; ++n) {
        cp_async_wait<1>();
        __syncthreads();                    // unit n landed (and, at n = 0, the mixed queries); all are done with unit n - 1
        if (n + 2 < n_units) load_unit(n + 2);
        cp_async_commit();
        int p = first_page + n / units_per_page, i = n % units_per_page;
        int key0 = p * LLMB_PAGE;
        if (key0 > warp_last_pos || key0 + LLMB_PAGE <= warp_oldest) continue;     // nothing of this page for this warp
        const __nv_bfloat16* tile_s = ring + (size_t)(n % STAGES) * TILE_ELEMS;
        if (i == 0) {
#pragma unroll
            for (int nb = 0; nb < 4; ++nb)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nb][e] = 0.f;
        }
        if (i < g_count) {
            const __nv_bfloat16* a_base = mixed + (size_t)(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldq + i * D + (lane >> 4) * 8;
#pragma unroll
            for (int kstep = 0; kstep < D / 16; ++kstep) {
                uint32_t a[4];
                ldmatrix_x4(a, a_base + kstep * 16);
#pragma unroll
                for (int nb = 0; nb < 4; nb += 2) {
                    uint32_t b[4];
                    int row = (half * 4 + nb) * 8 + (lane >> 4) * 8 + (lane & 7);
                    int col = kstep * 16 + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4(b, tile_s + row * LDS + col);
                    mma_bf16(s[nb], a[0], a[1], a[2], a[3], b[0], b[1]);
                    mma_bf16(s[nb + 1], a[0], a[1], a[2], a[3], b[2], b[3]);
                }
            }
            continue;
        }
        // the value tile: weights from the finished scores, then O += W V
        bool edge = key0 + LLMB_PAGE - 1 > start + tile * BQ + warp * 16 ||
                    (window > 0 && key0 < start + tile * BQ + warp * 16 + 15 - window + 1);
#pragma unroll
        for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float w0 = __frcp_rn(1.0f + fast_exp2(fmaf(s[nb][e], slope, offset)));
                float w1 = __frcp_rn(1.0f + fast_exp2(fmaf(s[nb][2 + e], slope, offset)));
                if (edge) {
                    int key = key0 + (half * 4 + nb) * 8 + 2 * t + e;
                    if (key > pos0 || key < low0) w0 = 0.f;
                    if (key > pos1 || key < low1) w1 = 0.f;
                }
                s[nb][e] = w0;
                s[nb][2 + e] = w1;
            }
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            uint32_t pa0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            uint32_t pa1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            uint32_t pa2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            uint32_t pa3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int n2 = 0; n2 < DV / 8; n2 += 2) {
                uint32_t b[4];
                int row = (half * 2 + kk) * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                int col = (n2 + (lane >> 4)) * 8;
                ldmatrix_x4_trans(b, tile_s + row * LDS + col);
                mma_bf16(acc[n2], pa0, pa1, pa2, pa3, b[0], b[1]);
                mma_bf16(acc[n2 + 1], pa0, pa1, pa2, pa3, b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();                            // the ring is free: the second halves' sums pass through it
    float* handover = reinterpret_cast<float*>(ring);          // [64 rows][DV]
    if (half == 1) {
#pragma unroll
        for (int n = 0; n < DV / 8; ++n) {
            float* to = handover + (size_t)(warp * 16 + g) * DV + n * 8 + 2 * t;
            to[0] = acc[n][0];
            to[1] = acc[n][1];
            to[8 * DV] = acc[n][2];
            to[8 * DV + 1] = acc[n][3];
        }
    }
    __syncthreads();
    if (half == 1) return;
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) {
        const float* from = handover + (size_t)(warp * 16 + g) * DV + n * 8 + 2 * t;
        acc[n][0] += from[0];
        acc[n][1] += from[1];
        acc[n][2] += from[8 * DV];
        acc[n][3] += from[8 * DV + 1];
    }

    __nv_bfloat16* o0 = out + (size_t)(first_token + row0) * out_stride + (size_t)head * DV;
    __nv_bfloat16* o1 = out + (size_t)(first_token + row1) * out_stride + (size_t)head * DV;
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) {
        if (row0 < n_new)
            *reinterpret_cast<__nv_bfloat162*>(o0 + n * 8 + 2 * t) = __floats2bfloat162_rn(acc[n][0] * out_scale, acc[n][1] * out_scale);
        if (row1 < n_new)
            *reinterpret_cast<__nv_bfloat162*>(o1 + n * 8 + 2 * t) = __floats2bfloat162_rn(acc[n][2] * out_scale, acc[n][3] * out_scale);
    }
}

template <int D, int DV>
static int launch_tiles(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* block_table,
                        int table_stride, int ring_pages, const int* cu_seqlens, const int* seq_lens, void* out,
                        int out_stride, int n_seqs, int max_new, int n_heads, int n_kv_heads, float scale, int window,
                        const float* talk, const float* head_bias, float out_scale, cudaStream_t stream) {
    constexpr int LDS = (D > DV ? D : DV) + PAD;
    int g_count = talk ? n_kv_heads : 1;
    size_t smem = sizeof(__nv_bfloat16) * ((size_t)BQ * (g_count * D + PAD) + (size_t)STAGES * LLMB_PAGE * LDS);
    LLMB_REQUIRE(smem <= 220 * 1024, "sigmoid_attention_tiles: %d key heads of %d do not fit in shared memory", g_count, D);
    static size_t configured = 0;
    if (smem > configured) {
        LLMB_CUDA(cudaFuncSetAttribute(sigmoid_attention_tiles_kernel<D, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem));
        configured = smem;
    }
    dim3 grid(n_heads, (max_new + BQ - 1) / BQ, n_seqs);
    sigmoid_attention_tiles_kernel<D, DV><<<grid, TILE_WARPS * 32, smem, stream>>>(
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_table,
        table_stride, ring_pages, cu_seqlens, seq_lens, (__nv_bfloat16*)out, out_stride, n_heads, n_kv_heads, scale, window,
        talk, head_bias, out_scale);
    return check_launch("sigmoid_attention_tiles");
}

// q: the new tokens' queries, packed sequence after sequence; token i of sequence b is row cu_seqlens[b] + i and
// stands at position seq_lens[b] - n_new(b) + i (seq_lens: the lengths after this step). max_new: the most new
// tokens any sequence brings.
LLMB_EXPORT int llmb_sigmoid_attention_tiles(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                             const int* block_table, int table_stride, int ring_pages,
                                             const int* cu_seqlens, const int* seq_lens, void* out, int out_stride,
                                             int n_seqs, int max_new, int n_heads, int n_kv_heads, int dim, int vdim,
                                             float scale, int window, const float* talk, const float* head_bias,
                                             float out_scale, cudaStream_t stream) {
    if (n_seqs == 0 || max_new == 0) return LLMB_OK;
    LLMB_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 && n_heads <= 65535,
                 "sigmoid_attention_tiles: %d heads are no multiple of %d kv heads", n_heads, n_kv_heads);
    LLMB_REQUIRE(n_seqs <= 65535 && max_new / BQ < 65535 && ring_pages > 0 && window >= 0, "sigmoid_attention_tiles: bad sizes");
    LLMB_REQUIRE(q_stride % 2 == 0 && out_stride % 2 == 0 && (reinterpret_cast<uintptr_t>(q) & 3) == 0 &&
                 (reinterpret_cast<uintptr_t>(out) & 3) == 0,
                 "sigmoid_attention_tiles: q and out must be 4-byte aligned with even row strides");
#define X(DK, DVAL)                                                                                                  \
    if (dim == DK && vdim == DVAL)                                                                                   \
        return launch_tiles<DK, DVAL>(q, q_stride, k_cache, v_cache, block_table, table_stride, ring_pages, cu_seqlens, \
                                      seq_lens, out, out_stride, n_seqs, max_new, n_heads, n_kv_heads, scale, window, \
                                      talk, head_bias, out_scale, stream);
    LLMB_SIGMOID_SHAPES(X)
#undef X
    return fail(LLMB_ERR_ARGUMENT, "sigmoid_attention_tiles: head size %d with value size %d is not built", dim, vdim);
}

// ----------------------------------------------------------------------------- one token a sequence

// sigmoid_attention_decode: a step in which every sequence brings one token is bound by reading the keys and
// values of the window once. A block serves one (slice of the pages, sequence) for ALL heads: the heads are the
// rows of the tensor-core tiles (16 * MT of them), the mixed queries of all heads lie in shared memory, and per
// page the G key tiles and the G value tiles stream through two buffers (two blocks share an SM). Each warp takes 16 of a
// page's 64 keys; the weights of a head go into the second product only with the value tile of the head's own
// group (the other rows of the operand are zero). Nothing is normalised, so the slices' results simply add: the
// four warps are added in a fixed order, and with more than one slice a second kernel adds the slices in order.
constexpr int DECODE_STAGES = 2;

// The mixed queries of a step of one token a sequence, once for all slices: mixed[seq][a][g * D + d] =
// sum over the heads b of group g of talk[a, b] * q[seq][b][d] (rows beyond the heads are zero).
__global__ void __launch_bounds__(128)
sigmoid_attention_mix_queries_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const float* __restrict__ talk,
                                     __nv_bfloat16* __restrict__ mixed, int rows, int n_heads, int n_kv_heads, int dim) {
    griddep_launch();
    griddep_wait();
    int seq = blockIdx.x, a = blockIdx.y;
    int group = n_heads / n_kv_heads, width = n_kv_heads * dim;
    const __nv_bfloat16* q_row = q + (size_t)seq * q_stride;
    __nv_bfloat16* to = mixed + ((size_t)seq * rows + a) * width;
    for (int c = threadIdx.x; c < width; c += 128) {
        int gi = c / dim, d = c % dim;
        float sum = 0.f;
        if (a < n_heads) {
            for (int b = 0; b < group; ++b) {
                int other = gi * group + b;
                float w = talk ? talk[(size_t)a * n_heads + other] : (other == a ? 1.f : 0.f);
                sum = fmaf(w, to_float(q_row[(size_t)other * dim + d]), sum);
            }
        }
        to[c] = __float2bfloat16_rn(sum);
    }
}

template <int D, int DV, int MT>
__global__ void __launch_bounds__(WARPS * 32)
sigmoid_attention_decode_kernel(const __nv_bfloat16* __restrict__ mixed_queries, const __nv_bfloat16* __restrict__ k_cache,
                                const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table,
                                int table_stride, int ring_pages, const int* __restrict__ seq_lens,
                                __nv_bfloat16* __restrict__ out, int out_stride, float* __restrict__ partial,
                                int n_heads, int n_kv_heads, float scale, int window,
                                const float* __restrict__ head_bias, float out_scale) {
    constexpr int LDS = (D > DV ? D : DV) + PAD;
    constexpr int TILE_ELEMS = LLMB_PAGE * LDS;
    constexpr int ROWS = 16 * MT;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    griddep_launch();
    griddep_wait();
    int split = blockIdx.x, n_splits = gridDim.x, seq = blockIdx.y;
    int group = n_heads / n_kv_heads;
    int g_count = n_kv_heads;
    int ldq = g_count * D + PAD;
    __nv_bfloat16* mixed = reinterpret_cast<__nv_bfloat16*>(smem_raw);     // [ROWS][ldq]
    __nv_bfloat16* ring = mixed + (size_t)ROWS * ldq;                       // [DECODE_STAGES][64][LDS]
    int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gl = lane >> 2, t = lane & 3;
    const int* pages = block_table + (size_t)seq * table_stride;
    int len = seq_lens[seq];
    int oldest = window > 0 ? max(len - window, 0) : 0;          // the query stands at len - 1
    int first_page = oldest / LLMB_PAGE, n_pages = (len + LLMB_PAGE - 1) / LLMB_PAGE;
    int per_split = (n_pages - first_page + n_splits - 1) / n_splits;
    int page_begin = min(first_page + split * per_split, n_pages), page_end = min(page_begin + per_split, n_pages);
    int units_per_page = 2 * g_count;
    int n_units = (page_end - page_begin) * units_per_page;

    auto load_unit = [&](int n) {
        int p = page_begin + n / units_per_page, i = n % units_per_page;
        size_t page = (size_t)pages[p % ring_pages];
        __nv_bfloat16* to = ring + (size_t)(n % DECODE_STAGES) * TILE_ELEMS;
        if (i < g_count) {
            const __nv_bfloat16* from = k_cache + ((page * n_kv_heads + i) * LLMB_PAGE) * D;
            for (int c = tid; c < LLMB_PAGE * (D / 8); c += WARPS * 32) {
                int row = c / (D / 8), col = (c % (D / 8)) * 8;
                cp_async16(to + row * LDS + col, from + (size_t)row * D + col);
            }
        } else {
            const __nv_bfloat16* from = v_cache + ((page * n_kv_heads + (i - g_count)) * LLMB_PAGE) * DV;
            for (int c = tid; c < LLMB_PAGE * (DV / 8); c += WARPS * 32) {
                int row = c / (DV / 8), col = (c % (DV / 8)) * 8;
                cp_async16(to + row * LDS + col, from + (size_t)row * DV + col);
            }
        }
    };
    {   // the sequence's mixed queries (made once a step by the kernel before this one) join the first group of copies
        int chunks = g_count * D / 8;
        const __nv_bfloat16* from = mixed_queries + (size_t)seq * ROWS * g_count * D;
        for (int c = tid; c < ROWS * chunks; c += WARPS * 32) {
            int row = c / chunks, col = (c % chunks) * 8;
            cp_async16(mixed + (size_t)row * ldq + col, from + (size_t)row * g_count * D + col);
        }
    }
#pragma unroll
    for (int n = 0; n < DECODE_STAGES - 1; ++n) {
        if (n < n_units) load_unit(n);
        cp_async_commit();
    }
    float slope = -scale * 1.4426950408889634f;
    float offset0[MT], offset1[MT];                  // -bias log2 e of this lane's two rows of every row tile
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        int h0 = mt * 16 + gl, h1 = h0 + 8;
        offset0[mt] = (head_bias && h0 < n_heads) ? -head_bias[h0] * 1.4426950408889634f : 0.f;
        offset1[mt] = (head_bias && h1 < n_heads) ? -head_bias[h1] * 1.4426950408889634f : 0.f;
    }

    float acc[MT][DV / 8][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int n = 0; n < DV / 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[mt][n][e] = 0.f;
    float s[MT][2][4];
    uint32_t pa[MT][4];

    for (int n = 0; n < n_units; ++n) {
        cp_async_wait<DECODE_STAGES - 2>();
        __syncthreads();                    // unit n landed (and, at n = 0, the mixed queries); all are done with unit n - 1
        if (n + DECODE_STAGES - 1 < n_units) load_unit(n + DECODE_STAGES - 1);
        cp_async_commit();
        int p = page_begin + n / units_per_page, i = n % units_per_page;
        int key_base = warp * 16;
        int first_key = p * LLMB_PAGE + key_base;
        if (first_key >= len || first_key + 16 <= oldest) continue;      // none of this warp's 16 keys is seen
        const __nv_bfloat16* tile_s = ring + (size_t)(n % DECODE_STAGES) * TILE_ELEMS;
        if (i == 0) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nb = 0; nb < 2; ++nb)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[mt][nb][e] = 0.f;
        }
        if (i < g_count) {
#pragma unroll
            for (int kstep = 0; kstep < D / 16; ++kstep) {
                uint32_t b[4];
                ldmatrix_x4(b, tile_s + (key_base + (lane >> 4) * 8 + (lane & 7)) * LDS + kstep * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    uint32_t a[4];
                    ldmatrix_x4(a, mixed + (size_t)(mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldq + i * D + kstep * 16 + (lane >> 4) * 8);
                    mma_bf16(s[mt][0], a[0], a[1], a[2], a[3], b[0], b[1]);
                    mma_bf16(s[mt][1], a[0], a[1], a[2], a[3], b[2], b[3]);
                }
            }
            if (i == g_count - 1) {                 // the scores are complete: the weights, as the second product's operand
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            int key = first_key + nb * 8 + 2 * t + e;
                            bool seen = key < len && key >= oldest;
                            float w0 = __frcp_rn(1.0f + fast_exp2(fmaf(s[mt][nb][e], slope, offset0[mt])));
                            float w1 = __frcp_rn(1.0f + fast_exp2(fmaf(s[mt][nb][2 + e], slope, offset1[mt])));
                            s[mt][nb][e] = seen ? w0 : 0.f;
                            s[mt][nb][2 + e] = seen ? w1 : 0.f;
                        }
                    pa[mt][0] = pack_bf16(s[mt][0][0], s[mt][0][1]);
                    pa[mt][1] = pack_bf16(s[mt][0][2], s[mt][0][3]);
                    pa[mt][2] = pack_bf16(s[mt][1][0], s[mt][1][1]);
                    pa[mt][3] = pack_bf16(s[mt][1][2], s[mt][1][3]);
                }
            }
            continue;
        }
        int gv = i - g_count;                       // the value tile of key/value head gv: only its group's rows
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            if (gv < (mt * 16) / group || gv > (mt * 16 + 15) / group) continue;       // no head of this row tile
            bool mine0 = (mt * 16 + gl) / group == gv, mine1 = (mt * 16 + gl + 8) / group == gv;
            uint32_t a0 = mine0 ? pa[mt][0] : 0u, a1 = mine1 ? pa[mt][1] : 0u;
            uint32_t a2 = mine0 ? pa[mt][2] : 0u, a3 = mine1 ? pa[mt][3] : 0u;
#pragma unroll
            for (int n2 = 0; n2 < DV / 8; n2 += 2) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, tile_s + (key_base + ((lane >> 3) & 1) * 8 + (lane & 7)) * LDS + (n2 + (lane >> 4)) * 8);
                mma_bf16(acc[mt][n2], a0, a1, a2, a3, b[0], b[1]);
                mma_bf16(acc[mt][n2 + 1], a0, a1, a2, a3, b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();                                // the buffers are free: the four warps' sums meet in them
    float* merge = reinterpret_cast<float*>(smem_raw);          // [WARPS][ROWS][DV]
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int n = 0; n < DV / 8; ++n) {
            float* to = merge + ((size_t)warp * ROWS + mt * 16 + gl) * DV + n * 8 + 2 * t;
            to[0] = acc[mt][n][0];
            to[1] = acc[mt][n][1];
            to[8 * DV] = acc[mt][n][2];
            to[8 * DV + 1] = acc[mt][n][3];
        }
    __syncthreads();
    for (int idx = tid; idx < n_heads * DV; idx += WARPS * 32) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v += merge[(size_t)w * ROWS * DV + idx];
        if (n_splits == 1) out[(size_t)seq * out_stride + idx] = __float2bfloat16_rn(v * out_scale);
        else partial[((size_t)seq * n_splits + split) * n_heads * DV + idx] = v;
    }
}

__global__ void sigmoid_attention_add_slices_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                                                    int out_stride, int width, int n_splits, float out_scale) {
    griddep_launch();
    griddep_wait();
    int seq = blockIdx.y;
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= width) return;
    float v = 0.f;
    for (int s = 0; s < n_splits; ++s) v += partial[((size_t)seq * n_splits + s) * width + idx];
    out[(size_t)seq * out_stride + idx] = __float2bfloat16_rn(v * out_scale);
}

template <int D, int DV, int MT>
static int launch_decode(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* block_table,
                         int table_stride, int ring_pages, const int* seq_lens, void* out, int out_stride, float* scratch,
                         int n_seqs, int n_heads, int n_kv_heads, float scale, int window, const float* talk,
                         const float* head_bias, float out_scale, int n_splits, cudaStream_t stream) {
    constexpr int LDS = (D > DV ? D : DV) + PAD;
    constexpr int ROWS = 16 * MT;
    size_t stream_bytes = sizeof(__nv_bfloat16) * ((size_t)ROWS * (n_kv_heads * D + PAD) + (size_t)DECODE_STAGES * LLMB_PAGE * LDS);
    size_t merge_bytes = sizeof(float) * WARPS * ROWS * DV;
    size_t smem = stream_bytes > merge_bytes ? stream_bytes : merge_bytes;
    LLMB_REQUIRE(smem <= 220 * 1024, "sigmoid_attention_decode: %d key heads of %d do not fit in shared memory", n_kv_heads, D);
    static size_t configured = 0;
    if (smem > configured) {
        LLMB_CUDA(cudaFuncSetAttribute(sigmoid_attention_decode_kernel<D, DV, MT>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    // the scratch begins with the mixed queries (bfloat16 [n_seqs][ROWS][kv heads * D]); the slices' sums follow
    __nv_bfloat16* mixed = reinterpret_cast<__nv_bfloat16*>(scratch);
    scratch += ((size_t)n_seqs * ROWS * n_kv_heads * D + 1) / 2;
    LLMB_CUDA(llmb::launch(sigmoid_attention_mix_queries_kernel, dim3(n_seqs, ROWS), dim3(128), 0, stream, true,
                           (const __nv_bfloat16*)q, q_stride, talk, mixed, ROWS, n_heads, n_kv_heads, D));
    LLMB_CUDA(llmb::launch(sigmoid_attention_decode_kernel<D, DV, MT>, dim3(n_splits, n_seqs), dim3(WARPS * 32), smem, stream,
                           true, (const __nv_bfloat16*)mixed, (const __nv_bfloat16*)k_cache,
                           (const __nv_bfloat16*)v_cache, block_table, table_stride, ring_pages, seq_lens,
                           (__nv_bfloat16*)out, out_stride, scratch, n_heads, n_kv_heads, scale, window, head_bias,
                           out_scale));
    if (n_splits > 1) {
        int width = n_heads * DV;
        LLMB_CUDA(llmb::launch(sigmoid_attention_add_slices_kernel, dim3(ceil_div(width, 256), n_seqs), dim3(256), 0, stream,
                               true, (const float*)scratch, (__nv_bfloat16*)out, out_stride, width, n_splits, out_scale));
    }
    return check_launch("sigmoid_attention_decode");
}

// One query a sequence (row b of q is sequence b's, at position seq_lens[b] - 1). scratch: the mixed queries
// (n_seqs * (16 or 32 rows) * n_kv_heads * dim bfloat16) and, where n_splits > 1, n_seqs * n_splits * n_heads * vdim
// floats. Up to 32 heads.
LLMB_EXPORT int llmb_sigmoid_attention_decode(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                              const int* block_table, int table_stride, int ring_pages,
                                              const int* seq_lens, void* out, int out_stride, float* scratch,
                                              long long scratch_floats, int n_seqs, int n_heads, int n_kv_heads, int dim,
                                              int vdim, float scale, int window, const float* talk,
                                              const float* head_bias, float out_scale, int n_splits, cudaStream_t stream) {
    if (n_seqs == 0) return LLMB_OK;
    LLMB_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 && n_heads <= 32,
                 "sigmoid_attention_decode: %d heads over %d kv heads (up to 32 heads)", n_heads, n_kv_heads);
    LLMB_REQUIRE(n_seqs <= 65535 && n_splits >= 1 && n_splits <= 65535 && ring_pages > 0 && window >= 0,
                 "sigmoid_attention_decode: bad sizes");
    long long mixed_floats = ((long long)n_seqs * (n_heads <= 16 ? 16 : 32) * n_kv_heads * dim + 1) / 2;
    LLMB_REQUIRE(scratch && scratch_floats >= mixed_floats + (n_splits > 1 ? (long long)n_seqs * n_splits * n_heads * vdim : 0),
                 "sigmoid_attention_decode: scratch too small");
#define X(DK, DVAL)                                                                                                   \
    if (dim == DK && vdim == DVAL) {                                                                                  \
        if (n_heads <= 16)                                                                                            \
            return launch_decode<DK, DVAL, 1>(q, q_stride, k_cache, v_cache, block_table, table_stride, ring_pages,  \
                                              seq_lens, out, out_stride, scratch, n_seqs, n_heads, n_kv_heads, scale, \
                                              window, talk, head_bias, out_scale, n_splits, stream);                  \
        return launch_decode<DK, DVAL, 2>(q, q_stride, k_cache, v_cache, block_table, table_stride, ring_pages,      \
                                          seq_lens, out, out_stride, scratch, n_seqs, n_heads, n_kv_heads, scale,     \
                                          window, talk, head_bias, out_scale, n_splits, stream);                      \
    }
    LLMB_SIGMOID_SHAPES(X)
#undef X
    return fail(LLMB_ERR_ARGUMENT, "sigmoid_attention_decode: head size %d with value size %d is not built", dim, vdim);
}

LLMB_PACKED(llmb_sigmoid_attention_generic)
LLMB_PACKED(llmb_sigmoid_attention_tiles)
LLMB_PACKED(llmb_sigmoid_attention_decode)
