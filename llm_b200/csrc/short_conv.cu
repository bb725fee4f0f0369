// A short causal convolution over time on every channel of a packed projection, with the state
// it carries from step to step, fused with what follows it in an attention mixer: the rotation of
// queries and keys and the write of keys and values into the paged cache.
//
//   y[t, c] = w[c, 0] u[p - (n - 1), c] + ... + w[c, n - 1] u[p, c],   n taps, p the position of token t,
//   u = 0 at negative positions
//
// u is the projection of the step's tokens [T, C] (queries | keys | values side by side). Values
// of positions before the step's first token come from the sequence's state [slots, taps - 1, C]:
// row i holds u at position start - (taps - 1) + i, zeros where that is negative (a slot's state is
// zeroed when the slot is taken). After the step the state holds the last taps - 1 rows again.
// With w == nullptr the projection passes through (a mixer without convolution). `w_rows` (optional):
// the same taps as bfloat16 [taps, C], where that copy is exact; the 16-byte kernel then reads a tap of
// eight channels in one load.
//
// Behind the convolution, per channel: the first n_rot elements of every unit of `rot_unit`
// channels of the query and key parts rotate by the angles of a 32-bit table [positions, n_rot]
// (cosines then sines; pairs (2i, 2i + 1) or (i, i + n_rot / 2)); queries leave as [T, Cq], keys
// go to the cache as rows of k_dim [pages, Hk, 64, k_dim], values as rows of v_dim
// [pages, Hv, 64, v_dim]. A key row may hold several rotated units (the maps of a differential
// attention: k_dim = 2 * rot_unit). Sums and angles are 32-bit; the result is rounded once.
//
// A token's position, sequence and slot come from device arrays, so a captured step replays.
#include "common.cuh"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_short_conv)

constexpr int MAX_TAPS = 16;                // the 16-byte kernel is built for up to 8

struct ConvArgs {
    const void* u; int u_stride;          // [T, C]
    const float* w; int taps;             // [C, taps] or nullptr
    const void* w_rows;                   // the same taps as bfloat16 [taps, C] (exact copies), or nullptr
    void* state;                          // [slots, taps - 1, C] or nullptr (taps == 1 or no convolution)
    const int* tok_pos; const int* tok_seq; const int* cu_seqlens; const int* seq_lens; const int* slot_ids;
    const float* table; int n_rot; int rot_unit; int interleaved;
    void* q_out; int q_width; int k_width; int v_width;
    const int* block_table; int table_stride; int ring_pages;
    void* k_cache; int k_heads; int k_dim;
    void* v_cache; int v_heads; int v_dim;
    int write_cache; int update_state;
    int n_tokens; int tile;               // the 16-byte kernel: tokens in all, and tokens a block walks
};

// The convolution's result for channel c of token t (32-bit).
template <typename T>
__device__ __forceinline__ float conv_value(const ConvArgs& a, int t, int c, int first_token, int pos, int start,
                                            const T* state_row, int channels) {
    const T* u = (const T*)a.u;
    if (a.w == nullptr) return to_float(u[(size_t)t * a.u_stride + c]);
    float sum = 0.f;
    const float* w = a.w + (size_t)c * a.taps;
    for (int j = 0; j < a.taps; ++j) {
        int p = pos - a.taps + 1 + j;                     // the position this tap reads
        float value;
        if (p >= start) value = to_float(u[(size_t)(first_token + (p - start)) * a.u_stride + c]);
        else {
            int row = (a.taps - 1) - (start - p);         // >= 0: start - p <= taps - 1
            value = to_float(state_row[(size_t)row * channels + c]);
        }
        sum = fmaf(w[j], value, sum);                     // taps in order: the same sum however the prompt was cut
    }
    return sum;
}

template <typename T>
__global__ void __launch_bounds__(256)
conv_rope_cache_kernel(ConvArgs a) {
    griddep_launch();
    griddep_wait();
    int t = blockIdx.x;
    int channels = a.q_width + a.k_width + a.v_width;
    int pos = a.tok_pos[t], b = a.tok_seq[t];
    int first_token = a.cu_seqlens[b];
    int start = pos - (t - first_token);                  // position of the sequence's first token in this step
    T* state_row = a.state ? (T*)a.state + (size_t)a.slot_ids[b] * (a.taps - 1) * channels : nullptr;
    int half = a.n_rot >> 1;
    size_t page = 0;
    int row = pos % LLMB_PAGE;
    if (a.write_cache) page = a.block_table[(size_t)b * a.table_stride + ((pos / LLMB_PAGE) % a.ring_pages)];
    const float* angles = a.table ? a.table + (size_t)pos * a.n_rot : nullptr;

    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        float y = conv_value<T>(a, t, c, first_token, pos, start, state_row, channels);
        bool is_q = c < a.q_width, is_k = !is_q && c < a.q_width + a.k_width;
        if ((is_q || is_k) && angles) {
            int local = is_q ? c : c - a.q_width;
            int d = local % a.rot_unit;                   // place inside the rotated unit
            if (d < a.n_rot) {
                int pair, partner;
                bool low;
                if (a.interleaved) { pair = d >> 1; low = (d & 1) == 0; partner = low ? c + 1 : c - 1; }
                else { low = d < half; pair = low ? d : d - half; partner = low ? c + half : c - half; }
                float other = conv_value<T>(a, t, partner, first_token, pos, start, state_row, channels);
                float cs = angles[pair], sn = angles[half + pair];
                y = low ? y * cs - other * sn : y * cs + other * sn;
            }
        }
        if (is_q) {
            ((T*)a.q_out)[(size_t)t * a.q_width + c] = from_float<T>(y);
        } else if (a.write_cache) {
            if (is_k) {
                int local = c - a.q_width, head = local / a.k_dim, d = local - head * a.k_dim;
                ((T*)a.k_cache)[((page * a.k_heads + head) * LLMB_PAGE + row) * a.k_dim + d] = from_float<T>(y);
            } else {
                int local = c - a.q_width - a.k_width, head = local / a.v_dim, d = local - head * a.v_dim;
                ((T*)a.v_cache)[((page * a.v_heads + head) * LLMB_PAGE + row) * a.v_dim + d] = from_float<T>(y);
            }
        }
    }
    // A sequence that brings one token is read by this block alone, every channel by one thread: the
    // thread that read a channel's state shifts it. (Longer pieces: conv_state_kernel, afterwards.)
    if (a.update_state && a.state && a.w) {
        __syncthreads();                                  // rotation partners have been read
        const T* u = (const T*)a.u;
        for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
            for (int i = 0; i + 1 < a.taps - 1; ++i) state_row[(size_t)i * channels + c] = state_row[(size_t)(i + 1) * channels + c];
            state_row[(size_t)(a.taps - 2) * channels + c] = u[(size_t)t * a.u_stride + c];
        }
    }
}

// The same work for bfloat16 with 16-byte accesses: a thread takes 8 neighbouring channels of a token.
// Needs every width, unit and rotated part to be a multiple of 8, pairs (2i, 2i + 1) (a pair then lies
// inside a thread's 8 channels) or no rotation, and 16-byte aligned rows. The thread that owns the
// channels also shifts their state in a decode step.
template <int TAPS>
__global__ void __launch_bounds__(256)
conv_rope_cache_vec_kernel(ConvArgs a) {
    griddep_launch();
    griddep_wait();
    using bf16 = __nv_bfloat16;
    int channels = a.q_width + a.k_width + a.v_width;
    int half = a.n_rot >> 1;
    const bf16* u = (const bf16*)a.u;
    int k_end = a.q_width + a.k_width;
    int t_begin = blockIdx.x * a.tile;
    int t_end = min(t_begin + a.tile, a.n_tokens);

    for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8; c < channels; c += gridDim.y * blockDim.x * 8) {
        // A block walks `tile` tokens. Where a token follows the one before in its sequence, the rows
        // held in registers move up by one and only the newest row is fetched.
        uint4 taps_raw[TAPS];                            // the rows of positions pos - TAPS + 1 .. pos, oldest first
        int prev_seq = -1, prev_pos = -2;
        bool is_q = c < a.q_width, is_k = !is_q && c < k_end;
        int rot_place = (is_q || is_k) ? (is_q ? c : c - a.q_width) % a.rot_unit : 0;
        bool rotates = (is_q || is_k) && a.table != nullptr && rot_place < a.n_rot;
        for (int t = t_begin; t < t_end; ++t) {
            int pos = a.tok_pos[t], b = a.tok_seq[t];
            bf16* state_row = nullptr;
            if (b == prev_seq && pos == prev_pos + 1) {
#pragma unroll
                for (int j = 0; j + 1 < TAPS; ++j) taps_raw[j] = taps_raw[j + 1];
                taps_raw[TAPS - 1] = *reinterpret_cast<const uint4*>(u + (size_t)t * a.u_stride + c);
            } else {
                int first_token = a.cu_seqlens[b];
                int start = pos - (t - first_token);
                if (a.state) state_row = (bf16*)a.state + (size_t)a.slot_ids[b] * (TAPS - 1) * channels;
#pragma unroll
                for (int j = 0; j < TAPS; ++j) {
                    int p = pos - TAPS + 1 + j;
                    const bf16* src = p >= start ? u + (size_t)(first_token + (p - start)) * a.u_stride + c
                                                 : state_row + (size_t)((TAPS - 1) - (start - p)) * channels + c;
                    taps_raw[j] = *reinterpret_cast<const uint4*>(src);
                }
            }
            prev_seq = b;
            prev_pos = pos;
            float y[8];
            if (a.w_rows) {                              // one coalesced 16-byte load a tap
#pragma unroll
                for (int e = 0; e < 8; ++e) y[e] = 0.f;
#pragma unroll
                for (int j = 0; j < TAPS; ++j) {
                    uint4 w_raw = *reinterpret_cast<const uint4*>((const bf16*)a.w_rows + (size_t)j * channels + c);
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        y[e] = fmaf(__bfloat162float(reinterpret_cast<const bf16*>(&w_raw)[e]),
                                    __bfloat162float(reinterpret_cast<const bf16*>(&taps_raw[j])[e]), y[e]);
                }
            } else if (a.w) {
                const float* w = a.w + (size_t)c * TAPS;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    float sum = 0.f;
#pragma unroll
                    for (int j = 0; j < TAPS; ++j)
                        sum = fmaf(w[e * TAPS + j], __bfloat162float(reinterpret_cast<const bf16*>(&taps_raw[j])[e]), sum);
                    y[e] = sum;
                }
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) y[e] = __bfloat162float(reinterpret_cast<const bf16*>(&taps_raw[TAPS - 1])[e]);
            }
            if (rotates) {
                const float* angles = a.table + (size_t)pos * a.n_rot;
                float4 cs = *reinterpret_cast<const float4*>(angles + (rot_place >> 1));
                float4 sn = *reinterpret_cast<const float4*>(angles + half + (rot_place >> 1));
                float cv[4] = {cs.x, cs.y, cs.z, cs.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float lo = y[2 * i], hi = y[2 * i + 1];
                    y[2 * i] = lo * cv[i] - hi * sv[i];
                    y[2 * i + 1] = hi * cv[i] + lo * sv[i];
                }
            }
            uint4 packed;
            __nv_bfloat162* out2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
            for (int i = 0; i < 4; ++i) out2[i] = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
            if (is_q) {
                *reinterpret_cast<uint4*>((bf16*)a.q_out + (size_t)t * a.q_width + c) = packed;
            } else if (a.write_cache) {
                size_t page = a.block_table[(size_t)b * a.table_stride + ((pos / LLMB_PAGE) % a.ring_pages)];
                int row = pos % LLMB_PAGE;
                if (is_k) {
                    int local = c - a.q_width, head = local / a.k_dim, d = local - head * a.k_dim;
                    *reinterpret_cast<uint4*>((bf16*)a.k_cache + ((page * a.k_heads + head) * LLMB_PAGE + row) * a.k_dim + d) = packed;
                } else {
                    int local = c - k_end, head = local / a.v_dim, d = local - head * a.v_dim;
                    *reinterpret_cast<uint4*>((bf16*)a.v_cache + ((page * a.v_heads + head) * LLMB_PAGE + row) * a.v_dim + d) = packed;
                }
            }
            if (a.update_state && TAPS > 1 && a.w) {     // one token of this sequence: the rows move up by one
#pragma unroll
                for (int j = 1; j < TAPS; ++j)
                    *reinterpret_cast<uint4*>(state_row + (size_t)(j - 1) * channels + c) = taps_raw[j];
            }
        }
    }
}

// The state after a step: the last taps - 1 rows of (old state rows, the step's rows). One block
// column per sequence; a thread owns a channel, reads its rows and then writes them.
template <typename T>
__global__ void __launch_bounds__(256)
conv_state_kernel(const T* __restrict__ u, int u_stride, T* __restrict__ state, int taps, int channels,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids) {
    griddep_launch();
    griddep_wait();
    int b = blockIdx.x;
    int first = cu_seqlens[b], count = cu_seqlens[b + 1] - first;
    int keep = taps - 1;
    T* rows = state + (size_t)slot_ids[b] * keep * channels;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        T held[MAX_TAPS];
        for (int i = 0; i < keep; ++i) {
            int from = i + count;                         // index into (old rows, new rows)
            held[i] = from < keep ? rows[(size_t)from * channels + c]
                                  : u[(size_t)(first + from - keep) * u_stride + c];
        }
        for (int i = 0; i < keep; ++i) rows[(size_t)i * channels + c] = held[i];
    }
}

LLMB_EXPORT int llmb_conv_rope_cache_write(
        const void* u, int u_stride, int dtype, const float* w, const void* w_rows, int taps, void* state,
        const int* tok_pos, const int* tok_seq, const int* cu_seqlens, const int* seq_lens, const int* slot_ids,
        const float* table, int n_rot, int rot_unit, int interleaved,
        void* q_out, int q_width, int k_width, int v_width,
        const int* block_table, int table_stride, int ring_pages,
        void* k_cache, int k_heads, int k_dim, void* v_cache, int v_heads, int v_dim,
        int write_cache, int n_tokens, int n_seqs, int single_tokens, cudaStream_t stream) {
    if (n_tokens == 0) return LLMB_OK;
    int channels = q_width + k_width + v_width;
    LLMB_REQUIRE(q_width > 0 && k_width >= 0 && v_width >= 0 && u_stride >= channels, "short_conv: bad widths");
    LLMB_REQUIRE(w == nullptr || (taps >= 1 && taps <= MAX_TAPS), "short_conv: %d taps (1 to %d are built)", taps, MAX_TAPS);
    LLMB_REQUIRE(w == nullptr || taps == 1 || state != nullptr, "short_conv: a convolution over time needs its state");
    LLMB_REQUIRE(table == nullptr || (n_rot > 0 && n_rot % 2 == 0 && rot_unit >= n_rot && q_width % rot_unit == 0 &&
                                      k_width % rot_unit == 0),
                 "short_conv: %d rotated elements do not fit units of %d", n_rot, rot_unit);
    LLMB_REQUIRE(!write_cache || (k_heads * k_dim == k_width && v_heads * v_dim == v_width && ring_pages > 0),
                 "short_conv: the cache rows do not fit the projection");
    ConvArgs a;
    a.u = u; a.u_stride = u_stride; a.w = w; a.w_rows = w ? w_rows : nullptr; a.taps = w ? taps : 1; a.state = (w && taps > 1) ? state : nullptr;
    a.tok_pos = tok_pos; a.tok_seq = tok_seq; a.cu_seqlens = cu_seqlens; a.seq_lens = seq_lens; a.slot_ids = slot_ids;
    a.table = table; a.n_rot = table ? n_rot : 0; a.rot_unit = rot_unit > 0 ? rot_unit : 1; a.interleaved = interleaved;
    a.q_out = q_out; a.q_width = q_width; a.k_width = k_width; a.v_width = v_width;
    a.block_table = block_table; a.table_stride = table_stride; a.ring_pages = ring_pages;
    a.k_cache = k_cache; a.k_heads = k_heads; a.k_dim = k_dim; a.v_cache = v_cache; a.v_heads = v_heads; a.v_dim = v_dim;
    a.write_cache = write_cache;
    a.update_state = single_tokens ? 1 : 0;
    a.n_tokens = n_tokens;
    a.tile = 1;
    // one block row per token; where a step has few tokens the channels are spread over block columns.
    // A block takes chunks of 256 neighbouring channels, so a pair (2i, 2i + 1) of units of even size never
    // leaves its block; a kernel that shifts the state itself AND rotates pairs that may lie in another
    // chunk must keep a token in one block (the partner's state row would be read by one block and
    // shifted by another).
    int columns = 1;
    if (!a.update_state || !a.state || !a.table || (a.interleaved && a.rot_unit % 2 == 0)) {
        columns = ceil_div(channels, 256);
        while (columns > 1 && (long long)n_tokens * columns > 148 * 8) columns = (columns + 1) / 2;
    }
    // 16-byte path: bfloat16, everything a multiple of 8 channels and aligned, pairs inside a thread's channels
    auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    bool vector = dtype == LLMB_DTYPE_BF16 && a.taps <= 8 && q_width % 8 == 0 && k_width % 8 == 0 && v_width % 8 == 0 && u_stride % 8 == 0 &&
                  aligned16(u) && aligned16(q_out) && aligned16(a.state) && aligned16(w) && aligned16(w_rows) &&
                  (!write_cache || (k_dim % 8 == 0 && v_dim % 8 == 0 && aligned16(k_cache) && aligned16(v_cache))) &&
                  (a.table == nullptr || (interleaved && n_rot % 8 == 0 && a.rot_unit % 8 == 0 && aligned16(table)));
    if (vector) {
        int vectors = channels / 8;
        // long steps: a block walks 8 tokens (a row is fetched once, not once a tap); short ones: a block a token
        a.n_tokens = n_tokens;
        a.tile = (!a.update_state && n_tokens >= 2048) ? 8 : 1;
        if (const char* forced = std::getenv("LLMB_CONV_TILE"))          // for measurements: force the tile
            if (!a.update_state && std::atoi(forced) > 0) a.tile = std::atoi(forced);
        int rows = ceil_div(n_tokens, a.tile);
        int cols = ceil_div(vectors, 256);
        while (cols > 1 && (long long)rows * cols > 148 * 16) cols = (cols + 1) / 2;
        dim3 vgrid(rows, cols);
        int threads = vectors < 256 ? ((vectors + 31) / 32) * 32 : 256;
        switch (a.taps) {
#define LLMB_CONV_CASE(N) case N: llmb::launch(conv_rope_cache_vec_kernel<N>, vgrid, threads, 0, stream, true, a); break;
            LLMB_CONV_CASE(1) LLMB_CONV_CASE(2) LLMB_CONV_CASE(3) LLMB_CONV_CASE(4)
            LLMB_CONV_CASE(5) LLMB_CONV_CASE(6) LLMB_CONV_CASE(7) LLMB_CONV_CASE(8)
#undef LLMB_CONV_CASE
        }
    } else {
        dim3 grid(n_tokens, columns);
        if (dtype == LLMB_DTYPE_F32) llmb::launch(conv_rope_cache_kernel<float>, grid, 256, 0, stream, true, a);
        else if (dtype == LLMB_DTYPE_BF16) llmb::launch(conv_rope_cache_kernel<__nv_bfloat16>, grid, 256, 0, stream, true, a);
        else return fail(LLMB_ERR_ARGUMENT, "short_conv: unknown dtype %d", dtype);
    }
    int code = check_launch("conv_rope_cache_write");
    if (code != LLMB_OK || a.state == nullptr || a.update_state) return code;
    dim3 state_grid(n_seqs, ceil_div(channels, 256) < 8 ? ceil_div(channels, 256) : 8);
    if (dtype == LLMB_DTYPE_F32)
        llmb::launch(conv_state_kernel<float>, state_grid, 256, 0, stream, true, (const float*)u, u_stride, (float*)state,
                     taps, channels, cu_seqlens, slot_ids);
    else
        llmb::launch(conv_state_kernel<__nv_bfloat16>, state_grid, 256, 0, stream, true, (const __nv_bfloat16*)u, u_stride,
                     (__nv_bfloat16*)state, taps, channels, cu_seqlens, slot_ids);
    return check_launch("conv_state");
}

// How many kernels one call launches (for the launch count of a step).
LLMB_EXPORT int llmb_conv_rope_cache_write_kernels(int has_conv, int taps, int single_tokens) {
    return (has_conv && taps > 1 && !single_tokens) ? 2 : 1;
}

LLMB_PACKED(llmb_conv_rope_cache_write)
