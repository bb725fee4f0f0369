// Differential attention over the paged cache: every query head holds two maps (two queries of
// `dim` elements against the two halves of a key row of 2 * dim), each map is a softmax attention of
// its own over the same values, and the head's result is
//
//   o = a1 - lambda * a2,   o <- o / sqrt(mean(o^2) + eps) * out_scale      (over the head's vdim values)
//
// with lambda one number of the layer. Which keys a query at position p sees: j <= p and
// (window == 0 or p - j < window or j < keep_first): a sliding window that also keeps the
// sequence's first tokens, at their true positions. Keys [pages, G, 64, 2 * dim], values
// [pages, G, 64, vdim]; query head h reads key/value head h / (H / G).
//
// This file holds the kernel for any sizes in 32-bit arithmetic: the kernel of the true 32-bit
// path and the fallback of the bfloat16 path. One block per (token, query head), four warps; warp w
// takes the visible keys number w, w + 4, ... (counted over the kept first tokens and then the
// window), the lanes spread over the head's elements; every warp keeps a running (max, sum,
// weighted values) per map, and the four partial results are merged in a fixed order. The order of
// reduction depends only on the query's position, so a token's result depends neither on the batch
// nor on how its prompt was cut.
#include "common.cuh"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_diff_attention)

constexpr int MAX_PER_LANE = LLMB_MAX_HEAD_DIM / 32;
constexpr int WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
diff_attention_generic_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                              const T* __restrict__ v_cache, const int* __restrict__ block_table,
                              int table_stride, int ring_pages, const int* __restrict__ tok_pos,
                              const int* __restrict__ tok_seq, T* __restrict__ out, int out_stride,
                              int n_heads, int n_kv_heads, int dim, int vdim, float scale, int window,
                              int keep_first, float lambda, float eps, float out_scale, int head_norm) {
    griddep_launch();
    griddep_wait();
    int t = blockIdx.x, head = blockIdx.y;
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int kv_head = head / (n_heads / n_kv_heads);
    int pos = tok_pos[t];
    const int* pages = block_table + (size_t)tok_seq[t] * table_stride;
    // visible keys: [0, kept) and [first, pos]
    int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    int kept = keep_first < first ? keep_first : first;
    int n_visible = kept + (pos - first + 1);

    float q1[MAX_PER_LANE], q2[MAX_PER_LANE], acc1[MAX_PER_LANE], acc2[MAX_PER_LANE];
    const T* q_row = q + (size_t)t * q_stride + (size_t)head * 2 * dim;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        int d = lane + 32 * i;
        q1[i] = d < dim ? to_float(q_row[d]) : 0.f;
        q2[i] = d < dim ? to_float(q_row[dim + d]) : 0.f;
        acc1[i] = acc2[i] = 0.f;
    }
    float max1 = -INFINITY, sum1 = 0.f, max2 = -INFINITY, sum2 = 0.f;

    for (int n = warp; n < n_visible; n += WARPS) {
        int j = n < kept ? n : first + (n - kept);
        int page = pages[(j / LLMB_PAGE) % ring_pages];
        size_t row = ((size_t)page * n_kv_heads + kv_head) * LLMB_PAGE + (j % LLMB_PAGE);
        const T* key = k_cache + row * 2 * dim;
        const T* value = v_cache + row * vdim;
        float dot1 = 0.f, dot2 = 0.f, vv[MAX_PER_LANE];
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            int d = lane + 32 * i;
            if (d < dim) {
                dot1 = fmaf(q1[i], to_float(key[d]), dot1);
                dot2 = fmaf(q2[i], to_float(key[dim + d]), dot2);
            }
            vv[i] = d < vdim ? to_float(value[d]) : 0.f;
        }
        float s1 = warp_sum(dot1) * scale, s2 = warp_sum(dot2) * scale;
        float new1 = fmaxf(max1, s1), new2 = fmaxf(max2, s2);
        float r1 = expf(max1 - new1), r2 = expf(max2 - new2);       // exp(-inf) = 0 on the first key
        float p1 = expf(s1 - new1), p2 = expf(s2 - new2);
        sum1 = sum1 * r1 + p1;
        sum2 = sum2 * r2 + p2;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            acc1[i] = fmaf(p1, vv[i], acc1[i] * r1);
            acc2[i] = fmaf(p2, vv[i], acc2[i] * r2);
        }
        max1 = new1;
        max2 = new2;
    }

    __shared__ float part_acc[2][WARPS][MAX_PER_LANE * 32];
    __shared__ float part_max[2][WARPS], part_sum[2][WARPS];
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        part_acc[0][warp][lane + 32 * i] = acc1[i];
        part_acc[1][warp][lane + 32 * i] = acc2[i];
    }
    if (lane == 0) {
        part_max[0][warp] = max1; part_sum[0][warp] = sum1;
        part_max[1][warp] = max2; part_sum[1][warp] = sum2;
    }
    __syncthreads();
    if (warp != 0) return;
    float weight[2][WARPS], denom[2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        float top = part_max[m][0];
#pragma unroll
        for (int w = 1; w < WARPS; ++w) top = fmaxf(top, part_max[m][w]);
        denom[m] = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            weight[m][w] = part_max[m][w] == -INFINITY ? 0.f : expf(part_max[m][w] - top);
            denom[m] += part_sum[m][w] * weight[m][w];
        }
    }
    float o[MAX_PER_LANE], square = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        int d = lane + 32 * i;
        float a1 = 0.f, a2 = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            a1 += part_acc[0][w][d] * weight[0][w];
            a2 += part_acc[1][w][d] * weight[1][w];
        }
        o[i] = d < vdim ? a1 / denom[0] - lambda * (a2 / denom[1]) : 0.f;
        square = fmaf(o[i], o[i], square);
    }
    float factor = out_scale;
    if (head_norm) factor *= 1.0f / sqrtf(warp_sum(square) / (float)vdim + eps);
    T* o_row = out + (size_t)t * out_stride + (size_t)head * vdim;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        int d = lane + 32 * i;
        if (d < vdim) o_row[d] = from_float<T>(o[i] * factor);
    }
}

LLMB_EXPORT int llmb_diff_attention_generic(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                            const int* block_table, int table_stride, int ring_pages,
                                            const int* tok_pos, const int* tok_seq, void* out, int out_stride,
                                            int dtype, int n_tokens, int n_heads, int n_kv_heads, int dim, int vdim,
                                            float scale, int window, int keep_first, float lambda, float eps,
                                            float out_scale, int head_norm, cudaStream_t stream) {
    if (n_tokens == 0) return LLMB_OK;
    LLMB_REQUIRE(dim > 0 && dim <= 32 * MAX_PER_LANE && vdim > 0 && vdim <= 32 * MAX_PER_LANE,
                 "diff_attention: head sizes %d / %d exceed %d", dim, vdim, 32 * MAX_PER_LANE);
    LLMB_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
                 "diff_attention: %d heads are no multiple of %d kv heads", n_heads, n_kv_heads);
    LLMB_REQUIRE(n_heads <= 65535 && ring_pages > 0 && window >= 0 && keep_first >= 0, "diff_attention: bad sizes");
    dim3 grid(n_tokens, n_heads);
    if (dtype == LLMB_DTYPE_F32)
        llmb::launch(diff_attention_generic_kernel<float>, grid, WARPS * 32, 0, stream, true,
                     (const float*)q, q_stride, (const float*)k_cache, (const float*)v_cache, block_table, table_stride,
                     ring_pages, tok_pos, tok_seq, (float*)out, out_stride, n_heads, n_kv_heads, dim, vdim, scale,
                     window, keep_first, lambda, eps, out_scale, head_norm);
    else if (dtype == LLMB_DTYPE_BF16)
        llmb::launch(diff_attention_generic_kernel<__nv_bfloat16>, grid, WARPS * 32, 0, stream, true,
                     (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                     block_table, table_stride, ring_pages, tok_pos, tok_seq, (__nv_bfloat16*)out, out_stride, n_heads,
                     n_kv_heads, dim, vdim, scale, window, keep_first, lambda, eps, out_scale, head_norm);
    else
        return fail(LLMB_ERR_ARGUMENT, "diff_attention: unknown dtype %d", dtype);
    return check_launch("diff_attention_generic");
}

LLMB_PACKED(llmb_diff_attention_generic)
