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
#include "common.cuh"

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

LLMB_PACKED(llmb_sigmoid_attention_generic)
