// Differential attention over the paged cache: every query head holds two maps (two queries of
// `dim` elements against the two halves of a key row of 2 * dim), each map is a softmax attention of
// its own over the same values, and the head's result is
//
//   o = a1 - lambda * a2,   o <- o / sqrt(mean(o^2) + eps) * out_scale      (over the head's vdim values)
//
// with lambda one number of the layer. Which keys a query at position p sees: j <= p and
// (window == 0 or p - j < window or j < keep_first): a sliding window beside which the sequence's
// first keep_first tokens stay visible, rotated and counted at the positions they have. Keys [pages, G, 64, 2 * dim], values
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

// =============================================================================================
// bfloat16 on the tensor cores (mma.sync.m16n8k16, 32-bit accumulation and softmax statistics).
// Map sizes DK and value sizes DV are multiples of 16 up to 128. Which pages a block walks: with a
// window only the pages that hold kept first tokens and the pages the window reaches, in that order;
// inside a page every score is masked by the rule at the top of this file.
// =============================================================================================
#include "mma.cuh"

constexpr int PAD = 8;                       // bf16 elements of row padding in shared memory

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The pages a range of query positions [first_pos, last_pos] sees: `sink_pages` pages from page 0, then
// pages first_page .. last_page.
struct PageWalk {
    int sink_pages, first_page, count;
    __device__ __forceinline__ int logical(int i) const { return i < sink_pages ? i : first_page + (i - sink_pages); }
};
__device__ __forceinline__ PageWalk page_walk(int first_pos, int last_pos, int window, int keep_first) {
    PageWalk w;
    int last_page = last_pos / LLMB_PAGE;
    w.first_page = 0;
    w.sink_pages = 0;
    if (window > 0) {
        int first_key = first_pos - window + 1;
        w.first_page = first_key > 0 ? first_key / LLMB_PAGE : 0;
        int sinks = keep_first > 0 ? (keep_first - 1) / LLMB_PAGE + 1 : 0;
        w.sink_pages = sinks < w.first_page ? sinks : w.first_page;
    }
    w.count = w.sink_pages + last_page - w.first_page + 1;
    return w;
}
__device__ __forceinline__ bool key_visible(int key, int pos, int window, int keep_first) {
    return key <= pos && (window == 0 || pos - key < window || key < keep_first);
}

// ----------------------------------------------------------------------------- prefill
// grid (heads, query tiles, sequences); tile 0 of the grid is a sequence's last 64 queries. Eight
// warps: warps 0-3 compute map 1 of the tile's 64 queries (16 rows a warp), warps 4-7 map 2, over
// the same pages of keys (a row holds both maps) and values in shared memory, two pages in
// flight. At the end the map-2 warps leave their result in shared memory and the map-1 warps form
// a1 - lambda a2, the head's norm and the scale, and store.
constexpr int PF_WARPS = 8;
constexpr int BQ = 64;
#ifndef LLMB_DIFF_PF_BLOCKS
#define LLMB_DIFF_PF_BLOCKS 2              // blocks an SM the prefill kernel is compiled for (128 registers a thread)
#endif

template <int DK, int DV>
__global__ void __launch_bounds__(PF_WARPS * 32, LLMB_DIFF_PF_BLOCKS)
diff_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ k_cache,
                    const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table,
                    int table_stride, int ring_pages, const int* __restrict__ cu_seqlens,
                    const int* __restrict__ seq_lens, __nv_bfloat16* __restrict__ out, int out_stride,
                    int n_heads, int n_kv_heads, float scale_log2, int window, int keep_first, float lambda,
                    float eps, float out_scale, int head_norm) {
    constexpr int LDK = 2 * DK + PAD, LDV = DV + PAD;
    constexpr int K_ELEMS = LLMB_PAGE * LDK, STAGE_ELEMS = K_ELEMS + LLMB_PAGE * LDV;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [2][keys 64 x LDK | values 64 x LDV]
    griddep_launch();
    griddep_wait();

    int seq = blockIdx.z, head = blockIdx.x;
    int first_token = cu_seqlens[seq];
    int n_new = cu_seqlens[seq + 1] - first_token;
    int n_tiles = (n_new + BQ - 1) / BQ;
    if ((int)blockIdx.y >= n_tiles) return;
    int tile = n_tiles - 1 - blockIdx.y;
    int start = seq_lens[seq] - n_new;
    int kv_head = head / (n_heads / n_kv_heads);
    int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    int map = warp >> 2, w4 = warp & 3;
    const int* pages = block_table + (size_t)seq * table_stride;

    int row0 = tile * BQ + w4 * 16 + g, row1 = row0 + 8;
    int pos0 = start + row0, pos1 = start + row1;
    int warp_first_pos = start + tile * BQ + w4 * 16;
    int warp_last_pos = start + min(tile * BQ + w4 * 16 + 15, n_new - 1);
    if (tile * BQ + w4 * 16 >= n_new) warp_last_pos = -1;
    int tile_first_pos = start + tile * BQ;
    int tile_last_pos = start + min(tile * BQ + BQ - 1, n_new - 1);
    PageWalk walk = page_walk(tile_first_pos, tile_last_pos, window, keep_first);

    uint32_t qa[DK / 16][4];
    {
        const __nv_bfloat16* q0 = q + (size_t)(first_token + row0) * q_stride + (size_t)(head * 2 + map) * DK;
        const __nv_bfloat16* q1 = q + (size_t)(first_token + row1) * q_stride + (size_t)(head * 2 + map) * DK;
        bool ok0 = row0 < n_new, ok1 = row1 < n_new;
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
            qa[ks][0] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * t) : 0u;
            qa[ks][1] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * t) : 0u;
            qa[ks][2] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + 2 * t) : 0u;
            qa[ks][3] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + 2 * t) : 0u;
        }
    }

    auto load_page = [&](int logical_page, int stage) {
        int page = pages[logical_page % ring_pages];
        size_t row_base = ((size_t)page * n_kv_heads + kv_head) * LLMB_PAGE;
        __nv_bfloat16* ks = smem + (size_t)stage * STAGE_ELEMS;
        __nv_bfloat16* vs = ks + K_ELEMS;
        constexpr int K_CHUNKS = 2 * DK / 8, V_CHUNKS = DV / 8;
        for (int c = tid; c < LLMB_PAGE * K_CHUNKS; c += PF_WARPS * 32) {
            int row = c / K_CHUNKS, col = (c % K_CHUNKS) * 8;
            cp_async16(ks + row * LDK + col, k_cache + (row_base + row) * (2 * DK) + col);
        }
        for (int c = tid; c < LLMB_PAGE * V_CHUNKS; c += PF_WARPS * 32) {
            int row = c / V_CHUNKS, col = (c % V_CHUNKS) * 8;
            cp_async16(vs + row * LDV + col, v_cache + (row_base + row) * DV + col);
        }
    };

    float acc[DV / 8][4];
#pragma unroll
    for (int n = 0; n < DV / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
    float max0 = -INFINITY, max1 = -INFINITY, sum0 = 0.f, sum1 = 0.f;

    load_page(walk.logical(0), 0);
    cp_async_commit();
    for (int p = 0; p < walk.count; ++p) {
        cp_async_wait<0>();
        __syncthreads();
        if (p + 1 < walk.count) load_page(walk.logical(p + 1), (p + 1) & 1);
        cp_async_commit();
        int key0 = walk.logical(p) * LLMB_PAGE;
        if (key0 > warp_last_pos) continue;                          // wholly above this warp's diagonal
        if (window > 0 && key0 >= keep_first && key0 + LLMB_PAGE - 1 < warp_first_pos - window + 1) continue;   // wholly before its windows

        const __nv_bfloat16* ks = smem + (size_t)(p & 1) * STAGE_ELEMS + map * DK;
        const __nv_bfloat16* vs = smem + (size_t)(p & 1) * STAGE_ELEMS + K_ELEMS;
        float s[8][4];
#pragma unroll
        for (int nb = 0; nb < 8; ++nb)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[nb][i] = 0.f;
#pragma unroll
        for (int kstep = 0; kstep < DK / 16; ++kstep) {
#pragma unroll
            for (int nb = 0; nb < 8; nb += 2) {
                uint32_t b[4];
                int row = nb * 8 + (lane >> 4) * 8 + (lane & 7);
                int col = kstep * 16 + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(b, ks + row * LDK + col);
                mma_bf16(s[nb], qa[kstep][0], qa[kstep][1], qa[kstep][2], qa[kstep][3], b[0], b[1]);
                mma_bf16(s[nb + 1], qa[kstep][0], qa[kstep][1], qa[kstep][2], qa[kstep][3], b[2], b[3]);
            }
        }
        // some key of the page may be hidden from some row of the warp: above the diagonal, or outside a window
        bool masked = key0 + LLMB_PAGE - 1 > warp_first_pos ||
                      (window > 0 && key0 < warp_last_pos + 16 - window + 1);
        float local0 = -INFINITY, local1 = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (masked) {
                    int key = key0 + nb * 8 + 2 * t + i;
                    if (!key_visible(key, pos0, window, keep_first)) s[nb][i] = -INFINITY;
                    if (!key_visible(key, pos1, window, keep_first)) s[nb][2 + i] = -INFINITY;
                }
                local0 = fmaxf(local0, s[nb][i]);
                local1 = fmaxf(local1, s[nb][2 + i]);
            }
        }
        local0 = fmaxf(local0, __shfl_xor_sync(0xffffffffu, local0, 1));
        local0 = fmaxf(local0, __shfl_xor_sync(0xffffffffu, local0, 2));
        local1 = fmaxf(local1, __shfl_xor_sync(0xffffffffu, local1, 1));
        local1 = fmaxf(local1, __shfl_xor_sync(0xffffffffu, local1, 2));
        // a row may have seen no key yet (its window starts later in this page's successors): its
        // maximum stays -inf, its probabilities are 0 and nothing is rescaled
        float new0 = fmaxf(max0, local0), new1 = fmaxf(max1, local1);
        float rescale0 = new0 == -INFINITY ? 1.f : fast_exp2((max0 - new0) * scale_log2);
        float rescale1 = new1 == -INFINITY ? 1.f : fast_exp2((max1 - new1) * scale_log2);
        max0 = new0;
        max1 = new1;
        float shift0 = new0 == -INFINITY ? 0.f : new0 * scale_log2, shift1 = new1 == -INFINITY ? 0.f : new1 * scale_log2;
        float add0 = 0.f, add1 = 0.f;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                s[nb][i] = fast_exp2(fmaf(s[nb][i], scale_log2, -shift0));
                s[nb][2 + i] = fast_exp2(fmaf(s[nb][2 + i], scale_log2, -shift1));
                add0 += s[nb][i];
                add1 += s[nb][2 + i];
            }
        }
        sum0 = sum0 * rescale0 + add0;
        sum1 = sum1 * rescale1 + add1;
#pragma unroll
        for (int n = 0; n < DV / 8; ++n) {
            acc[n][0] *= rescale0; acc[n][1] *= rescale0;
            acc[n][2] *= rescale1; acc[n][3] *= rescale1;
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t pa0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            uint32_t pa1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            uint32_t pa2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            uint32_t pa3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int n = 0; n < DV / 8; n += 2) {
                uint32_t b[4];
                int row = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                int col = (n + (lane >> 4)) * 8;
                ldmatrix_x4_trans(b, vs + row * LDV + col);
                mma_bf16(acc[n], pa0, pa1, pa2, pa3, b[0], b[1]);
                mma_bf16(acc[n + 1], pa0, pa1, pa2, pa3, b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();                                   // the page buffers are free: map 2 passes its result through them

    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    float inv0 = 1.0f / sum0, inv1 = 1.0f / sum1;       // every stored row sees at least its own key
    float* second = reinterpret_cast<float*>(smem_raw);             // [64][DV] of map 2
    int local0_row = w4 * 16 + g, local1_row = local0_row + 8;
    if (map == 1) {
#pragma unroll
        for (int n = 0; n < DV / 8; ++n) {
            *reinterpret_cast<float2*>(second + local0_row * DV + n * 8 + 2 * t) = make_float2(acc[n][0] * inv0, acc[n][1] * inv0);
            *reinterpret_cast<float2*>(second + local1_row * DV + n * 8 + 2 * t) = make_float2(acc[n][2] * inv1, acc[n][3] * inv1);
        }
    }
    __syncthreads();
    if (map == 1) return;
    float square0 = 0.f, square1 = 0.f;
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) {
        float2 b0 = *reinterpret_cast<const float2*>(second + local0_row * DV + n * 8 + 2 * t);
        float2 b1 = *reinterpret_cast<const float2*>(second + local1_row * DV + n * 8 + 2 * t);
        acc[n][0] = acc[n][0] * inv0 - lambda * b0.x;
        acc[n][1] = acc[n][1] * inv0 - lambda * b0.y;
        acc[n][2] = acc[n][2] * inv1 - lambda * b1.x;
        acc[n][3] = acc[n][3] * inv1 - lambda * b1.y;
        square0 = fmaf(acc[n][0], acc[n][0], fmaf(acc[n][1], acc[n][1], square0));
        square1 = fmaf(acc[n][2], acc[n][2], fmaf(acc[n][3], acc[n][3], square1));
    }
    float factor0 = out_scale, factor1 = out_scale;
    if (head_norm) {
        square0 += __shfl_xor_sync(0xffffffffu, square0, 1);
        square0 += __shfl_xor_sync(0xffffffffu, square0, 2);
        square1 += __shfl_xor_sync(0xffffffffu, square1, 1);
        square1 += __shfl_xor_sync(0xffffffffu, square1, 2);
        factor0 *= 1.0f / sqrtf(square0 / (float)DV + eps);
        factor1 *= 1.0f / sqrtf(square1 / (float)DV + eps);
    }
    __nv_bfloat16* o0 = out + (size_t)(first_token + row0) * out_stride + (size_t)head * DV;
    __nv_bfloat16* o1 = out + (size_t)(first_token + row1) * out_stride + (size_t)head * DV;
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) {
        if (row0 < n_new)
            *reinterpret_cast<__nv_bfloat162*>(o0 + n * 8 + 2 * t) = __floats2bfloat162_rn(acc[n][0] * factor0, acc[n][1] * factor0);
        if (row1 < n_new)
            *reinterpret_cast<__nv_bfloat162*>(o1 + n * 8 + 2 * t) = __floats2bfloat162_rn(acc[n][2] * factor1, acc[n][3] * factor1);
    }
}

// ----------------------------------------------------------------------------- decode
// One new query per sequence. grid (slices, kv heads, sequences); a block serves one (sequence, kv
// head) over a slice of the pages the query sees. The query heads of the group are rows 0-7 of the
// tensor-core tile for map 1 and rows 8-15 for map 2: two products against the two halves of a key
// row give both maps' scores in one accumulator, and one product P V gives both maps' weighted
// values. Four warps take 16 keys of a page each; the warps, then the slices (a second kernel),
// are merged in a fixed order, and the merge forms a1 - lambda a2, the head's norm and the scale.
constexpr int DC_WARPS = 4;
// Pages in a block's ring. A launch of few blocks (up to two an SM) takes as many as fit in about 110 KB,
// between 3 and 8: small pages need more of them in flight to keep HBM busy. A launch of many blocks takes
// 3, so that more blocks share an SM (measured at maps of 32 and values of 64, context 8,192: batch 8
// 945 -> 846 us a step with the deep ring, batch 64 2,108 -> 2,475 us).
template <int DK, int DV>
__host__ __device__ constexpr int decode_stages() {
    constexpr int bytes = LLMB_PAGE * (2 * DK + PAD + DV + PAD) * 2;
    constexpr int fit = (110 * 1024) / bytes;
    return fit < 3 ? 3 : fit > 8 ? 8 : fit;
}

template <int DV>
__device__ __forceinline__ void diff_finish(float* a1, const float* a2, float lambda, float eps, float out_scale,
                                            int head_norm, __nv_bfloat16* o, int lane) {
    // a1, a2 [DV] in shared memory (32-bit); one warp
    float square = 0.f;
    for (int d = lane; d < DV; d += 32) {
        float v = a1[d] - lambda * a2[d];
        a1[d] = v;
        square = fmaf(v, v, square);
    }
    float factor = out_scale;
    if (head_norm) factor *= 1.0f / sqrtf(warp_sum(square) / (float)DV + eps);
    for (int d = lane; d < DV; d += 32) o[d] = __float2bfloat16_rn(a1[d] * factor);
}

// partials: acc [seq, head, map, slice, DV], stats [seq, head, map, slice, 2] = (max in base-2 units, sum)
template <int DK, int DV, int DC_STAGES>
__global__ void __launch_bounds__(DC_WARPS * 32)
diff_decode_split_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ k_cache,
                         const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table,
                         int table_stride, int ring_pages, const int* __restrict__ seq_lens,
                         const int* __restrict__ seq_order, float* __restrict__ part_acc,
                         float* __restrict__ part_stats, __nv_bfloat16* __restrict__ out, int out_stride,
                         int n_heads, int n_kv_heads, float scale_log2, int window, int keep_first, float lambda,
                         float eps, float out_scale, int head_norm) {
    constexpr int LDK = 2 * DK + PAD, LDV = DV + PAD;
    constexpr int K_ELEMS = LLMB_PAGE * LDK, STAGE_ELEMS = K_ELEMS + LLMB_PAGE * LDV;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    griddep_launch();
    int split = blockIdx.x, n_splits = gridDim.x, kv_head = blockIdx.y;
    int seq = seq_order ? seq_order[blockIdx.z] : (int)blockIdx.z;
    int group = n_heads / n_kv_heads;
    int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    int len = seq_lens[seq], pos = len - 1;
    PageWalk walk = page_walk(pos, pos, window, keep_first);
    int per_split = (walk.count + n_splits - 1) / n_splits;
    int begin = min(split * per_split, walk.count), end = min(begin + per_split, walk.count);
    int n_my = end - begin;
    const int* pages = block_table + (size_t)seq * table_stride;
    int newest_page = pos / LLMB_PAGE;

    auto load_page = [&](int logical_page, int stage) {
        int page = pages[logical_page % ring_pages];
        size_t row_base = ((size_t)page * n_kv_heads + kv_head) * LLMB_PAGE;
        __nv_bfloat16* ks = smem + (size_t)stage * STAGE_ELEMS;
        __nv_bfloat16* vs = ks + K_ELEMS;
        constexpr int K_CHUNKS = 2 * DK / 8, V_CHUNKS = DV / 8;
        for (int c = tid; c < LLMB_PAGE * K_CHUNKS; c += DC_WARPS * 32) {
            int row = c / K_CHUNKS, col = (c % K_CHUNKS) * 8;
            cp_async16(ks + row * LDK + col, k_cache + (row_base + row) * (2 * DK) + col);
        }
        for (int c = tid; c < LLMB_PAGE * V_CHUNKS; c += DC_WARPS * 32) {
            int row = c / V_CHUNKS, col = (c % V_CHUNKS) * 8;
            cp_async16(vs + row * LDV + col, v_cache + (row_base + row) * DV + col);
        }
    };
    // The kernel before this one writes the queries and the newest position of the cache; every older
    // page is final. The first pages of the slice are requested before griddep_wait(), except the
    // page of the newest position.
    int late = -1;
#pragma unroll
    for (int s = 0; s < DC_STAGES - 1; ++s) {
        if (s < n_my) {
            if (walk.logical(begin + s) == newest_page) late = s;
            else load_page(walk.logical(begin + s), s);
        }
        cp_async_commit();
    }
    griddep_wait();
    if (late >= 0) {
        load_page(newest_page, late);
        cp_async_commit();
    }

    // A fragments: rows 0-7 map 1 of head kv_head * group + g, rows 8-15 map 2 of the same head
    uint32_t qa0[DK / 16], qa1[DK / 16], qa2[DK / 16], qa3[DK / 16];
    {
        const __nv_bfloat16* q_row = q + (size_t)seq * q_stride + (size_t)(kv_head * group + g) * 2 * DK;
        bool valid = g < group;
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
            qa0[ks] = valid ? *reinterpret_cast<const uint32_t*>(q_row + ks * 16 + 2 * t) : 0u;
            qa2[ks] = valid ? *reinterpret_cast<const uint32_t*>(q_row + ks * 16 + 8 + 2 * t) : 0u;
            qa1[ks] = valid ? *reinterpret_cast<const uint32_t*>(q_row + DK + ks * 16 + 2 * t) : 0u;
            qa3[ks] = valid ? *reinterpret_cast<const uint32_t*>(q_row + DK + ks * 16 + 8 + 2 * t) : 0u;
        }
    }
    float acc[DV / 8][4];
#pragma unroll
    for (int n = 0; n < DV / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
    float max0 = -INFINITY, max1 = -INFINITY, sum0 = 0.f, sum1 = 0.f;     // map 1 (row g), map 2 (row g + 8)

    for (int i = 0; i < n_my; ++i) {
        if (late >= 0 && i >= n_my - (DC_STAGES - 1)) cp_async_wait<0>();   // the late page was committed last
        else cp_async_wait<DC_STAGES - 2>();
        __syncthreads();
        if (i + DC_STAGES - 1 < n_my) load_page(walk.logical(begin + i + DC_STAGES - 1), (i + DC_STAGES - 1) % DC_STAGES);
        cp_async_commit();
        const __nv_bfloat16* ks = smem + (size_t)(i % DC_STAGES) * STAGE_ELEMS;
        const __nv_bfloat16* vs = ks + K_ELEMS;
        int key_base = warp * 16;
        int first_key = walk.logical(begin + i) * LLMB_PAGE + key_base;
        int key[4] = {first_key + 2 * t, first_key + 2 * t + 1, first_key + 8 + 2 * t, first_key + 9 + 2 * t};
        bool seen[4];
        bool any = false;
#pragma unroll
        for (int j = 0; j < 4; ++j) { seen[j] = key_visible(key[j], pos, window, keep_first); any = any || seen[j]; }
        if (!__any_sync(0xffffffffu, any)) continue;         // none of this warp's 16 keys is visible

        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int kstep = 0; kstep < DK / 16; ++kstep) {
            uint32_t b[4], c[4];
            int row = key_base + (lane >> 4) * 8 + (lane & 7);
            int col = kstep * 16 + ((lane >> 3) & 1) * 8;
            ldmatrix_x4(b, ks + row * LDK + col);                  // map 1's half of the key rows
            ldmatrix_x4(c, ks + row * LDK + DK + col);             // map 2's half
            mma_bf16(s0, qa0[kstep], 0u, qa2[kstep], 0u, b[0], b[1]);
            mma_bf16(s1, qa0[kstep], 0u, qa2[kstep], 0u, b[2], b[3]);
            mma_bf16(s0, 0u, qa1[kstep], 0u, qa3[kstep], c[0], c[1]);
            mma_bf16(s1, 0u, qa1[kstep], 0u, qa3[kstep], c[2], c[3]);
        }
        // s0: keys first_key + 2t, +1; s1: keys first_key + 8 + 2t, +1; [0..1] map 1 (row g), [2..3] map 2 (row g + 8)
        float v0[4] = {s0[0], s0[1], s1[0], s1[1]}, v1[4] = {s0[2], s0[3], s1[2], s1[3]};
        float local0 = -INFINITY, local1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v0[j] = seen[j] ? v0[j] * scale_log2 : -INFINITY;
            v1[j] = seen[j] ? v1[j] * scale_log2 : -INFINITY;
            local0 = fmaxf(local0, v0[j]);
            local1 = fmaxf(local1, v1[j]);
        }
        local0 = fmaxf(local0, __shfl_xor_sync(0xffffffffu, local0, 1));
        local0 = fmaxf(local0, __shfl_xor_sync(0xffffffffu, local0, 2));
        local1 = fmaxf(local1, __shfl_xor_sync(0xffffffffu, local1, 1));
        local1 = fmaxf(local1, __shfl_xor_sync(0xffffffffu, local1, 2));
        float new0 = fmaxf(max0, local0), new1 = fmaxf(max1, local1);     // finite: a key of the warp is visible
        float rescale0 = exp2f(max0 - new0), rescale1 = exp2f(max1 - new1);
        float p0[4], p1[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) { p0[j] = exp2f(v0[j] - new0); p1[j] = exp2f(v1[j] - new1); }
        sum0 = sum0 * rescale0 + (p0[0] + p0[1] + p0[2] + p0[3]);
        sum1 = sum1 * rescale1 + (p1[0] + p1[1] + p1[2] + p1[3]);
        max0 = new0;
        max1 = new1;
        uint32_t pa0 = pack_bf16(p0[0], p0[1]), pa1 = pack_bf16(p1[0], p1[1]);
        uint32_t pa2 = pack_bf16(p0[2], p0[3]), pa3 = pack_bf16(p1[2], p1[3]);
#pragma unroll
        for (int n = 0; n < DV / 8; ++n) {
            acc[n][0] *= rescale0; acc[n][1] *= rescale0;
            acc[n][2] *= rescale1; acc[n][3] *= rescale1;
        }
#pragma unroll
        for (int n = 0; n < DV / 8; n += 2) {
            uint32_t b[4];
            int row = key_base + ((lane >> 3) & 1) * 8 + (lane & 7);
            int col = (n + (lane >> 4)) * 8;
            ldmatrix_x4_trans(b, vs + row * LDV + col);
            mma_bf16(acc[n], pa0, pa1, pa2, pa3, b[0], b[1]);
            mma_bf16(acc[n + 1], pa0, pa1, pa2, pa3, b[2], b[3]);
        }
    }
    cp_async_wait<0>();
    __syncthreads();                                 // the stage buffers are free: reuse them

    // merge the four warps: rows 0-7 map 1, rows 8-15 map 2 of the group's heads
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    float* merge_acc = reinterpret_cast<float*>(smem_raw);            // [WARPS][16][DV]
    float* merge_max = merge_acc + DC_WARPS * 16 * DV;                // [WARPS][16]
    float* merge_sum = merge_max + DC_WARPS * 16;
    float* merged = merge_sum + DC_WARPS * 16;                        // [16][DV]
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) {
        *reinterpret_cast<float2*>(merge_acc + (warp * 16 + g) * DV + n * 8 + 2 * t) = make_float2(acc[n][0], acc[n][1]);
        *reinterpret_cast<float2*>(merge_acc + (warp * 16 + 8 + g) * DV + n * 8 + 2 * t) = make_float2(acc[n][2], acc[n][3]);
    }
    if (t == 0) {
        merge_max[warp * 16 + g] = max0; merge_sum[warp * 16 + g] = sum0;
        merge_max[warp * 16 + 8 + g] = max1; merge_sum[warp * 16 + 8 + g] = sum1;
    }
    __syncthreads();
    for (int idx = tid; idx < 2 * group * DV; idx += DC_WARPS * 32) {
        int which = idx / (group * DV), rest = idx - which * group * DV;
        int head = rest / DV, d = rest - head * DV, row = which * 8 + head;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < DC_WARPS; ++w) m = fmaxf(m, merge_max[w * 16 + row]);
        float value = 0.f, sum = 0.f;
#pragma unroll
        for (int w = 0; w < DC_WARPS; ++w) {
            float mw = merge_max[w * 16 + row];
            float weight = mw == -INFINITY ? 0.f : exp2f(mw - m);
            value += merge_acc[(w * 16 + row) * DV + d] * weight;
            sum += merge_sum[w * 16 + row] * weight;
        }
        if (n_splits == 1) {
            merged[row * DV + d] = value / sum;
        } else {
            size_t slot = (((size_t)seq * n_heads + kv_head * group + head) * 2 + which) * n_splits + split;
            part_acc[slot * DV + d] = value;
            if (d == 0) { part_stats[slot * 2] = m; part_stats[slot * 2 + 1] = sum; }
        }
    }
    if (n_splits > 1) return;
    __syncthreads();
    for (int head = warp; head < group; head += DC_WARPS)
        diff_finish<DV>(merged + head * DV, merged + (8 + head) * DV, lambda, eps, out_scale, head_norm,
                        out + (size_t)seq * out_stride + (size_t)(kv_head * group + head) * DV, lane);
}

// One block (two warps: one per map, then warp 0 finishes) per (head, sequence).
template <int DV>
__global__ void __launch_bounds__(64)
diff_decode_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_stats,
                           __nv_bfloat16* __restrict__ out, int out_stride, int n_heads, int n_splits, float lambda,
                           float eps, float out_scale, int head_norm) {
    griddep_launch();
    griddep_wait();
    __shared__ float maps[2][DV];
    int seq = blockIdx.y, head = blockIdx.x, which = threadIdx.x >> 5, lane = threadIdx.x & 31;
    size_t base = (((size_t)seq * n_heads + head) * 2 + which) * n_splits;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_stats[(base + s) * 2]);
    for (int d = lane; d < DV; d += 32) {
        float value = 0.f, sum = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            float ms = part_stats[(base + s) * 2];
            float weight = ms == -INFINITY ? 0.f : exp2f(ms - m);
            value += part_acc[(base + s) * DV + d] * weight;
            sum += part_stats[(base + s) * 2 + 1] * weight;
        }
        maps[which][d] = value / sum;
    }
    __syncthreads();
    if (which == 0)
        diff_finish<DV>(maps[0], maps[1], lambda, eps, out_scale, head_norm,
                        out + (size_t)seq * out_stride + (size_t)head * DV, lane);
}

template <int DK, int DV>
static int launch_prefill(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* block_table,
                          int table_stride, int ring_pages, const int* cu_seqlens, const int* seq_lens, void* out,
                          int out_stride, int n_seqs, int max_new, int n_heads, int n_kv_heads, float scale, int window,
                          int keep_first, float lambda, float eps, float out_scale, int head_norm, cudaStream_t stream) {
    size_t stage_bytes = (size_t)2 * LLMB_PAGE * (2 * DK + PAD + DV + PAD) * sizeof(__nv_bfloat16);
    size_t pass_bytes = (size_t)BQ * DV * sizeof(float);
    size_t smem = stage_bytes > pass_bytes ? stage_bytes : pass_bytes;
    static bool configured = false;
    if (!configured) {
        LLMB_CUDA(cudaFuncSetAttribute(diff_prefill_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    dim3 grid(n_heads, (max_new + BQ - 1) / BQ, n_seqs);
    llmb::launch(diff_prefill_kernel<DK, DV>, grid, PF_WARPS * 32, smem, stream, true,
                 (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                 block_table, table_stride, ring_pages, cu_seqlens, seq_lens, (__nv_bfloat16*)out, out_stride, n_heads,
                 n_kv_heads, scale * 1.4426950408889634f, window, keep_first, lambda, eps, out_scale, head_norm);
    return check_launch("diff_attention_prefill");
}

template <int DK, int DV>
static int launch_decode(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* block_table,
                         int table_stride, int ring_pages, const int* seq_lens, const int* seq_order, void* out,
                         int out_stride, float* scratch, int n_seqs, int n_heads, int n_kv_heads, float scale, int window,
                         int keep_first, float lambda, float eps, float out_scale, int head_norm, int n_splits,
                         cudaStream_t stream) {
    constexpr int DEEP = decode_stages<DK, DV>();
    bool deep = DEEP > 3 && (long long)n_splits * n_kv_heads * n_seqs <= 2 * 148;
    int stages = deep ? DEEP : 3;
    size_t stage_bytes = (size_t)stages * LLMB_PAGE * (2 * DK + PAD + DV + PAD) * sizeof(__nv_bfloat16);
    size_t merge_bytes = (size_t)(DC_WARPS * 16 * DV + 2 * DC_WARPS * 16 + 16 * DV) * sizeof(float);
    size_t smem = stage_bytes > merge_bytes ? stage_bytes : merge_bytes;
    static bool configured = false;
    if (!configured) {
        size_t most = (size_t)DEEP * LLMB_PAGE * (2 * DK + PAD + DV + PAD) * sizeof(__nv_bfloat16);
        most = most > merge_bytes ? most : merge_bytes;
        LLMB_CUDA(cudaFuncSetAttribute(diff_decode_split_kernel<DK, DV, DEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most));
        LLMB_CUDA(cudaFuncSetAttribute(diff_decode_split_kernel<DK, DV, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most));
        configured = true;
    }
    float* part_acc = scratch;
    float* part_stats = scratch + (size_t)n_seqs * n_heads * 2 * n_splits * DV;
    dim3 grid(n_splits, n_kv_heads, n_seqs);
#define LLMB_DIFF_DECODE(STAGES)                                                                                       \
    llmb::launch(diff_decode_split_kernel<DK, DV, STAGES>, grid, DC_WARPS * 32, smem, stream, true,                      \
                 (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,      \
                 block_table, table_stride, ring_pages, seq_lens, seq_order, part_acc, part_stats, (__nv_bfloat16*)out, \
                 out_stride, n_heads, n_kv_heads, scale * 1.4426950408889634f, window, keep_first, lambda, eps,         \
                 out_scale, head_norm)
    if (deep) LLMB_DIFF_DECODE(DEEP); else LLMB_DIFF_DECODE(3);
#undef LLMB_DIFF_DECODE
    int code = check_launch("diff_attention_decode_split");
    if (code || n_splits == 1) return code;
    llmb::launch(diff_decode_combine_kernel<DV>, dim3(n_heads, n_seqs), 64, 0, stream, true, (const float*)part_acc,
                 (const float*)part_stats, (__nv_bfloat16*)out, out_stride, n_heads, n_splits, lambda, eps, out_scale,
                 head_norm);
    return check_launch("diff_attention_decode_combine");
}

LLMB_EXPORT int llmb_diff_attention_tc_supports(int n_heads, int n_kv_heads, int dim, int vdim, int decode) {
    LLMB_REQUIRE(n_kv_heads > 0 && n_heads % n_kv_heads == 0, "diff_attention: %d heads are no multiple of %d kv heads",
                 n_heads, n_kv_heads);
    LLMB_REQUIRE(!decode || n_heads / n_kv_heads <= 8, "diff_attention_decode: a group of %d query heads exceeds 8",
                 n_heads / n_kv_heads);
#define X(DK, DV) if (dim == DK && vdim == DV) return LLMB_OK;
    LLMB_DIFF_SHAPES(X)
#undef X
    return fail(LLMB_ERR_ARGUMENT, "diff_attention: map size %d with value size %d (served: 32/32, 32/64, 48/96, 64/64, "
                "64/128, 128/128)", dim, vdim);
}

LLMB_EXPORT int llmb_diff_attention_prefill(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                            const int* block_table, int table_stride, int ring_pages,
                                            const int* cu_seqlens, const int* seq_lens, void* out, int out_stride,
                                            int n_seqs, int max_new, int n_heads, int n_kv_heads, int dim, int vdim,
                                            float scale, int window, int keep_first, float lambda, float eps,
                                            float out_scale, int head_norm, cudaStream_t stream) {
    if (n_seqs == 0 || max_new == 0) return LLMB_OK;
    int code = llmb_diff_attention_tc_supports(n_heads, n_kv_heads, dim, vdim, 0);
    if (code) return code;
    LLMB_REQUIRE(n_seqs <= 65535 && max_new / BQ < 65535 && ring_pages > 0 && window >= 0 && keep_first >= 0 && scale > 0.f,
                 "diff_attention_prefill: bad sizes");
    LLMB_REQUIRE(q_stride % 8 == 0 && out_stride % 2 == 0 && (reinterpret_cast<uintptr_t>(q) & 3) == 0 &&
                 (reinterpret_cast<uintptr_t>(out) & 3) == 0 && (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(v_cache) & 15) == 0,
                 "diff_attention_prefill: q and out must be 4-byte aligned, the cache 16-byte aligned");
#define X(DK, DV)                                                                                                     \
    if (dim == DK && vdim == DV)                                                                                       \
        return launch_prefill<DK, DV>(q, q_stride, k_cache, v_cache, block_table, table_stride, ring_pages, cu_seqlens, \
                                      seq_lens, out, out_stride, n_seqs, max_new, n_heads, n_kv_heads, scale, window,   \
                                      keep_first, lambda, eps, out_scale, head_norm, stream);
    LLMB_DIFF_SHAPES(X)
#undef X
    return fail(LLMB_ERR_ARGUMENT, "diff_attention_prefill: no kernel");
}

LLMB_EXPORT long long llmb_diff_attention_decode_scratch_floats(int n_seqs, int n_heads, int vdim, int n_splits) {
    return (long long)n_seqs * n_heads * 2 * n_splits * (vdim + 2);
}

LLMB_EXPORT int llmb_diff_attention_decode(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                           const int* block_table, int table_stride, int ring_pages,
                                           const int* seq_lens, const int* seq_order, void* out, int out_stride,
                                           float* scratch, long long scratch_floats, int n_seqs, int n_heads,
                                           int n_kv_heads, int dim, int vdim, float scale, int window, int keep_first,
                                           float lambda, float eps, float out_scale, int head_norm, int n_splits,
                                           cudaStream_t stream) {
    if (n_seqs == 0) return LLMB_OK;
    int code = llmb_diff_attention_tc_supports(n_heads, n_kv_heads, dim, vdim, 1);
    if (code) return code;
    LLMB_REQUIRE(n_splits >= 1 && n_splits <= 65535 && n_seqs <= 65535 && ring_pages > 0 && window >= 0 &&
                 keep_first >= 0 && scale > 0.f, "diff_attention_decode: bad sizes");
    LLMB_REQUIRE(q_stride % 2 == 0 && (reinterpret_cast<uintptr_t>(q) & 3) == 0 &&
                 (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_cache) & 15) == 0,
                 "diff_attention_decode: q must be 4-byte aligned with an even row stride, the cache 16-byte aligned");
    LLMB_REQUIRE(n_splits == 1 || (scratch != nullptr && scratch_floats >= llmb_diff_attention_decode_scratch_floats(
                                                                               n_seqs, n_heads, vdim, n_splits)),
                 "diff_attention_decode: scratch too small");
#define X(DK, DV)                                                                                                    \
    if (dim == DK && vdim == DV)                                                                                      \
        return launch_decode<DK, DV>(q, q_stride, k_cache, v_cache, block_table, table_stride, ring_pages, seq_lens,  \
                                     seq_order, out, out_stride, scratch, n_seqs, n_heads, n_kv_heads, scale, window, \
                                     keep_first, lambda, eps, out_scale, head_norm, n_splits, stream);
    LLMB_DIFF_SHAPES(X)
#undef X
    return fail(LLMB_ERR_ARGUMENT, "diff_attention_decode: no kernel");
}

LLMB_PACKED(llmb_diff_attention_prefill)
LLMB_PACKED(llmb_diff_attention_decode)
