// A real-gated linear recurrence behind a short causal convolution (the recurrent block of De et al.,
// "Griffin"), on C channels cut into `blocks` equal parts of P = C / blocks:
//
//     u[t, c]  = conv_b[c] + sum_j conv_w[c, j] * x[t - (taps - 1) + j, c]       (x = 0 before a sequence's start)
//     r[t, c]  = sigmoid(gate_a_bias[c] + sum_i gate_a[b, c - bP, i] * u[t, bP + i])     b = c / P
//     i[t, c]  = sigmoid(gate_i_bias[c] + sum_i gate_i[b, c - bP, i] * u[t, bP + i])
//     a        = exp(rate[c] * r)                                                  (rate = -decay * softplus(lam) < 0)
//     S[t, c]  = a * S[t - 1, c] + sqrt(1 - a^2) * i * u                           (S = 0 before the start)
//     out[t, c] = out_scale * S[t, c] * gelu(y[t, c])                              (tanh form of gelu)
//
// x and y are the two branches' projections (with their biases) in the run's dtype. Everything between
// reading them and rounding `out` is 32-bit: the convolution's sum, both gates' matrix products (on the
// CUDA cores, fixed order of summation per output), the decay, the recurrence and S.
//
// Per sequence the cache holds state[slot] = [taps, C] float32: rows 0 .. taps - 2 are the last taps - 1
// inputs x (oldest first), the last row is S. A slot's state is zeroed when the slot is taken, which is
// the convolution's zero padding and S = 0 for a sequence's first token: nothing treats it specially.
//
// Three kernels. conv: u of every token and channel, once, from x and the state (a value is `taps`
// multiply-adds; neighbouring threads take neighbouring channels). gates: tiles of 128 (long steps) or
// 32 tokens x 64 channels of one part over u; a thread owns 8 (or 2) tokens x 4 channels of both gates, so
// that 16 multiply-adds ride on every 16-byte read of shared memory; every output sums its inputs in
// rising order, whatever the tile; it writes a and the driving term sqrt(1 - a^2) i u of every token.
// scan: one thread per (sequence, channel) walks the sequence's tokens of this step in order, 16 at a
// time with the next 16 tokens' values already requested (the chain S <- a S + b is the only thing
// that has to wait), then brings the state up to date (S, and the last taps - 1 inputs). The first
// kernel only reads the state, the last writes it.
//
// Long steps (more than SCAN_SERIAL tokens) scan in three passes over chunks of 64 packed tokens, so that
// the tokens of a long prompt are not walked one after the other by a single thread: `scan_local` forms
// every chunk's product of a and its end value from a zero start (a sequence's first token of the step
// takes its S from the state there and stops the carry: a = 0), `scan_carry` walks the chunks in order
// (S at a chunk's start), `scan_apply` walks each chunk again from that start and writes the results, the
// new S of sequences that end in it and their convolution rows. The sums are the same up to rounding
// (a chunk's start value is formed from the chunk before it as a whole); short steps, and so every decode
// step, keep the token order exactly.
#include "common.cuh"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_gated_recurrence)

constexpr int MAX_TAPS = 16;
constexpr int TN = 64;        // output channels of a tile
constexpr int KC = 16;        // input channels staged at a time
constexpr int SCAN_THREADS = 64;
constexpr int SCAN_AHEAD = 16;
constexpr int SCAN_SERIAL = 256;   // steps of up to this many tokens are scanned by one thread a (sequence, channel)
constexpr int SCAN_CHUNK = 64;

// Where the convolution finds its inputs: the tokens of the same sequence in this step, and before the
// step's first token the rows of the state.
template <typename T>
struct ConvSource {
    const T* x;
    int x_stride;
    const float* state;       // [slots, taps, C]
    const float* conv_w;      // [C, taps]
    const float* conv_b;
    int taps, channels;

    __device__ __forceinline__ float value(int t, int seq_start, int slot, int c) const {
        float sum = conv_b[c];
        for (int j = 0; j < taps; ++j) {
            int src = t - (taps - 1) + j;
            float in = src >= seq_start ? to_float(x[(size_t)src * x_stride + c])
                                        : state[((size_t)slot * taps + (taps - 1 + src - seq_start)) * channels + c];
            sum = fmaf(conv_w[(size_t)c * taps + j], in, sum);
        }
        return sum;
    }
};

template <typename T>
__global__ void __launch_bounds__(256)
conv_kernel(ConvSource<T> source, const int* __restrict__ tok_seq, const int* __restrict__ cu_seqlens,
            const int* __restrict__ slot_ids, float* __restrict__ u) {
    griddep_launch();
    griddep_wait();
    int t = blockIdx.x;
    int c = blockIdx.y * 256 + threadIdx.x;
    if (c >= source.channels) return;
    int seq = tok_seq[t];
    u[(size_t)t * source.channels + c] = source.value(t, cu_seqlens[seq], slot_ids[seq], c);
}

// TT: tokens a thread owns; a tile has 16 * TT tokens.
template <int TT>
__global__ void __launch_bounds__(256)
gates_kernel(const float* __restrict__ u, int channels, const float* __restrict__ gate_a, const float* __restrict__ gate_a_bias,
                  const float* __restrict__ gate_i, const float* __restrict__ gate_i_bias, int part,
                  const float* __restrict__ rate, float* __restrict__ decay, float* __restrict__ drive, int n_tokens) {
    constexpr int TM = 16 * TT;
    // rows padded by four floats: a thread's 16-byte reads stay aligned, and the stores (16 neighbouring threads
    // write one column) spread over the banks
    __shared__ __align__(16) float u_tile[KC][TM + 4];      // [input channel][token]
    __shared__ __align__(16) float a_tile[KC][TN + 4];      // [input channel][output channel]
    __shared__ __align__(16) float i_tile[KC][TN + 4];
    griddep_launch();
    griddep_wait();
    int tiles_per_part = (part + TN - 1) / TN;
    int b = blockIdx.y / tiles_per_part;                 // which part of the channels
    int o0 = (blockIdx.y % tiles_per_part) * TN;         // first output of the tile, inside the part
    int t0 = blockIdx.x * TM;
    // thread (ty, tx) owns tokens ty * TT .. + TT - 1 and outputs tx * 4 .. + 3
    int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc_a[TT][4], acc_i[TT][4];
#pragma unroll
    for (int m = 0; m < TT; ++m)
#pragma unroll
        for (int n = 0; n < 4; ++n) acc_a[m][n] = acc_i[m][n] = 0.f;
    const float* wa = gate_a + (size_t)b * part * part;
    const float* wi = gate_i + (size_t)b * part * part;
    // the next chunk's values are requested into registers before this chunk's products run
    constexpr int U_PER = TM * KC / 256, W_PER = TN * KC / 256;
    float u_next[U_PER], a_next[W_PER], i_next[W_PER];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int j = 0; j < U_PER; ++j) {
            int e = threadIdx.x + j * 256;
            int m = e / KC, k = e % KC;                 // neighbouring threads: neighbouring channels of one token
            int t = t0 + m;
            u_next[j] = (t < n_tokens && k0 + k < part) ? u[(size_t)t * channels + b * part + k0 + k] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < W_PER; ++j) {
            int e = threadIdx.x + j * 256;
            int n = e / KC, k = e % KC;                 // neighbouring threads: neighbouring inputs of one output row
            bool live = o0 + n < part && k0 + k < part;
            size_t at = (size_t)(o0 + n) * part + k0 + k;
            a_next[j] = live ? wa[at] : 0.f;
            i_next[j] = live ? wi[at] : 0.f;
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < part; k0 += KC) {
#pragma unroll
        for (int j = 0; j < U_PER; ++j) {
            int e = threadIdx.x + j * 256;
            u_tile[e % KC][e / KC] = u_next[j];
        }
#pragma unroll
        for (int j = 0; j < W_PER; ++j) {
            int e = threadIdx.x + j * 256;
            a_tile[e % KC][e / KC] = a_next[j];
            i_tile[e % KC][e / KC] = i_next[j];
        }
        __syncthreads();
        if (k0 + KC < part) fetch(k0 + KC);
#pragma unroll
        for (int k = 0; k < KC; ++k) {
            float un[TT];
            if (TT % 4 == 0) {
#pragma unroll
                for (int m = 0; m < TT; m += 4) {
                    float4 v = *reinterpret_cast<const float4*>(&u_tile[k][ty * TT + m]);
                    un[m] = v.x; un[m + 1] = v.y; un[m + 2] = v.z; un[m + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int m = 0; m < TT; ++m) un[m] = u_tile[k][ty * TT + m];
            }
            float4 av = *reinterpret_cast<const float4*>(&a_tile[k][tx * 4]);
            float4 iv = *reinterpret_cast<const float4*>(&i_tile[k][tx * 4]);
            float an[4] = {av.x, av.y, av.z, av.w}, in[4] = {iv.x, iv.y, iv.z, iv.w};
#pragma unroll
            for (int m = 0; m < TT; ++m)
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    acc_a[m][n] = fmaf(an[n], un[m], acc_a[m][n]);
                    acc_i[m][n] = fmaf(in[n], un[m], acc_i[m][n]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int m = 0; m < TT; ++m) {
        int t = t0 + ty * TT + m;
        if (t >= n_tokens) continue;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            int o = o0 + tx * 4 + n;
            if (o >= part) continue;
            int c = b * part + o;
            float uc = u[(size_t)t * channels + c];
            float r = 1.0f / (1.0f + expf(-(acc_a[m][n] + gate_a_bias[c])));
            float g = 1.0f / (1.0f + expf(-(acc_i[m][n] + gate_i_bias[c])));
            float a = expf(rate[c] * r);
            decay[(size_t)t * channels + c] = a;
            drive[(size_t)t * channels + c] = sqrtf(1.0f - a * a) * g * uc;
        }
    }
}

template <typename T>
__device__ __forceinline__ void update_conv_rows(float* rows, int taps, int channels, const T* x, int x_stride,
                                                 int first, int count, int c);

__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_kernel(const T* __restrict__ y, int y_stride, const T* __restrict__ x, int x_stride,
            const float* __restrict__ decay, const float* __restrict__ drive, float* __restrict__ state, int taps,
            int channels, const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids, T* __restrict__ out,
            int out_stride, float out_scale) {
    griddep_launch();
    griddep_wait();
    int c = blockIdx.x * SCAN_THREADS + threadIdx.x;
    if (c >= channels) return;
    int seq = blockIdx.y;
    int first = cu_seqlens[seq], last = cu_seqlens[seq + 1];
    if (first >= last) return;
    float* rows = state + (size_t)slot_ids[seq] * taps * channels + c;      // row r at rows[r * channels]
    float s = rows[(size_t)(taps - 1) * channels];
    // the values of SCAN_AHEAD tokens are held while those of the next SCAN_AHEAD are on their way
    float a_now[SCAN_AHEAD], b_now[SCAN_AHEAD], y_now[SCAN_AHEAD], a_next[SCAN_AHEAD], b_next[SCAN_AHEAD], y_next[SCAN_AHEAD];
    auto fetch = [&](int t0, float (&a)[SCAN_AHEAD], float (&b)[SCAN_AHEAD], float (&g)[SCAN_AHEAD]) {
#pragma unroll
        for (int i = 0; i < SCAN_AHEAD; ++i) {
            int t = t0 + i;
            bool live = t < last;
            a[i] = live ? decay[(size_t)t * channels + c] : 0.f;
            b[i] = live ? drive[(size_t)t * channels + c] : 0.f;
            g[i] = live ? to_float(y[(size_t)t * y_stride + c]) : 0.f;
        }
    };
    fetch(first, a_now, b_now, y_now);
    for (int t0 = first; t0 < last; t0 += SCAN_AHEAD) {
        fetch(t0 + SCAN_AHEAD, a_next, b_next, y_next);
#pragma unroll
        for (int i = 0; i < SCAN_AHEAD; ++i) {
            int t = t0 + i;
            if (t < last) {
                s = fmaf(a_now[i], s, b_now[i]);
                out[(size_t)t * out_stride + c] = from_float<T>(s * gelu_tanh(y_now[i]) * out_scale);
            }
        }
#pragma unroll
        for (int i = 0; i < SCAN_AHEAD; ++i) { a_now[i] = a_next[i]; b_now[i] = b_next[i]; y_now[i] = y_next[i]; }
    }
    rows[(size_t)(taps - 1) * channels] = s;
    update_conv_rows(rows, taps, channels, x, x_stride, first, last - first, c);
}

// The last taps - 1 inputs of a sequence after a step of `count` tokens that began at packed token `first`: row r
// of the new state is input (count - (taps - 1) + r) of this step, or, where that lies before the step, row
// (r + count) of the old state. rows: the sequence's state at this channel, row r at rows[r * channels].
template <typename T>
__device__ __forceinline__ void update_conv_rows(float* rows, int taps, int channels, const T* x, int x_stride,
                                                 int first, int count, int c) {
    float old[MAX_TAPS];
#pragma unroll
    for (int r = 0; r < MAX_TAPS; ++r) old[r] = (r < taps - 1) ? rows[(size_t)r * channels] : 0.f;
#pragma unroll
    for (int r = 0; r < MAX_TAPS; ++r) {
        if (r >= taps - 1) break;
        int src = count - (taps - 1) + r;
        float v;
        if (src >= 0) {
            v = to_float(x[(size_t)(first + src) * x_stride + c]);
        } else {
            v = 0.f;
#pragma unroll
            for (int q = 0; q < MAX_TAPS; ++q) if (q == r + count) v = old[q];
        }
        rows[(size_t)r * channels] = v;
    }
}

// A step in which every sequence brings one token: token b is sequence b's, nothing is walked.
template <typename T>
__global__ void __launch_bounds__(256)
scan_single_kernel(const T* __restrict__ y, int y_stride, const T* __restrict__ x, int x_stride,
                   const float* __restrict__ decay, const float* __restrict__ drive, float* __restrict__ state, int taps,
                   int channels, const int* __restrict__ slot_ids, T* __restrict__ out, int out_stride, float out_scale) {
    griddep_launch();
    griddep_wait();
    int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= channels) return;
    int t = blockIdx.y;
    float* rows = state + (size_t)slot_ids[t] * taps * channels + c;
    float s = fmaf(decay[(size_t)t * channels + c], rows[(size_t)(taps - 1) * channels], drive[(size_t)t * channels + c]);
    out[(size_t)t * out_stride + c] = from_float<T>(s * gelu_tanh(to_float(y[(size_t)t * y_stride + c])) * out_scale);
    rows[(size_t)(taps - 1) * channels] = s;
    for (int r = 0; r + 1 < taps - 1; ++r) rows[(size_t)r * channels] = rows[(size_t)(r + 1) * channels];
    if (taps > 1) rows[(size_t)(taps - 2) * channels] = to_float(x[(size_t)t * x_stride + c]);
}

// Pass 1 of the chunked scan. A sequence's first token of the step becomes a token without a carry: its
// driving term takes a * S(state) in, its a becomes 0 (both rewritten in place).
__global__ void __launch_bounds__(SCAN_THREADS)
scan_local_kernel(float* __restrict__ decay, float* __restrict__ drive, const float* __restrict__ state, int taps,
                  int channels, const int* __restrict__ tok_seq, const int* __restrict__ cu_seqlens,
                  const int* __restrict__ slot_ids, float* __restrict__ products, float* __restrict__ ends, int n_tokens) {
    griddep_launch();
    griddep_wait();
    int c = blockIdx.x * SCAN_THREADS + threadIdx.x;
    if (c >= channels) return;
    int chunk = blockIdx.y, t0 = chunk * SCAN_CHUNK, t1 = min(t0 + SCAN_CHUNK, n_tokens);
    float product = 1.f, s = 0.f;
    for (int t = t0; t < t1; ++t) {
        float a = decay[(size_t)t * channels + c], b = drive[(size_t)t * channels + c];
        int seq = tok_seq[t];
        if (t == cu_seqlens[seq]) {
            b = fmaf(a, state[((size_t)slot_ids[seq] * taps + taps - 1) * channels + c], b);
            a = 0.f;
            decay[(size_t)t * channels + c] = a;
            drive[(size_t)t * channels + c] = b;
        }
        product *= a;
        s = fmaf(a, s, b);
    }
    products[(size_t)chunk * channels + c] = product;
    ends[(size_t)chunk * channels + c] = s;
}

// Pass 2: ends[k] becomes S at the START of chunk k.
__global__ void __launch_bounds__(SCAN_THREADS)
scan_carry_kernel(const float* __restrict__ products, float* __restrict__ ends, int channels, int n_chunks) {
    griddep_launch();
    griddep_wait();
    int c = blockIdx.x * SCAN_THREADS + threadIdx.x;
    if (c >= channels) return;
    float s = 0.f;
    for (int k = 0; k < n_chunks; ++k) {
        float p = products[(size_t)k * channels + c], e = ends[(size_t)k * channels + c];
        ends[(size_t)k * channels + c] = s;
        s = fmaf(p, s, e);
    }
}

// Pass 3: each chunk again from its start value; results, and the state of the sequences that end here.
template <typename T>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_apply_kernel(const T* __restrict__ y, int y_stride, const T* __restrict__ x, int x_stride,
                  const float* __restrict__ decay, const float* __restrict__ drive, const float* __restrict__ starts,
                  float* __restrict__ state, int taps, int channels, const int* __restrict__ tok_seq,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids, T* __restrict__ out,
                  int out_stride, float out_scale, int n_tokens) {
    griddep_launch();
    griddep_wait();
    int c = blockIdx.x * SCAN_THREADS + threadIdx.x;
    if (c >= channels) return;
    int chunk = blockIdx.y, t0 = chunk * SCAN_CHUNK, t1 = min(t0 + SCAN_CHUNK, n_tokens);
    float s = starts[(size_t)chunk * channels + c];
    for (int t = t0; t < t1; ++t) {
        s = fmaf(decay[(size_t)t * channels + c], s, drive[(size_t)t * channels + c]);
        out[(size_t)t * out_stride + c] = from_float<T>(s * gelu_tanh(to_float(y[(size_t)t * y_stride + c])) * out_scale);
        int seq = tok_seq[t];
        if (t + 1 == cu_seqlens[seq + 1]) {              // the sequence's last token of the step
            float* rows = state + (size_t)slot_ids[seq] * taps * channels + c;
            rows[(size_t)(taps - 1) * channels] = s;
            int first = cu_seqlens[seq];
            update_conv_rows(rows, taps, channels, x, x_stride, first, t + 1 - first, c);
        }
    }
}

// work [3, T, C] float32: u, a, the driving term.
LLMB_EXPORT int llmb_gated_recurrence(const void* y, int y_stride, const void* x, int x_stride, int dtype,
                                      const float* conv_w, const float* conv_b, int taps, const float* gate_a,
                                      const float* gate_a_bias, const float* gate_i, const float* gate_i_bias,
                                      int blocks, const float* rate, float* state, const int* tok_seq,
                                      const int* cu_seqlens, const int* slot_ids, void* out, int out_stride,
                                      float out_scale, float* work, int n_tokens, int channels, int n_seqs,
                                      int single_tokens, cudaStream_t stream) {
    if (n_tokens == 0) return LLMB_OK;
    LLMB_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "gated_recurrence: %d taps (1 to %d are built)", taps, MAX_TAPS);
    LLMB_REQUIRE(channels > 0 && blocks > 0 && channels % blocks == 0 && n_seqs > 0,
                 "gated_recurrence: %d channels in %d parts", channels, blocks);
    int part = channels / blocks;
    bool long_step = n_tokens > 64;                 // the result is the same either way
    dim3 grid_gates(ceil_div(n_tokens, long_step ? 128 : 32), blocks * ceil_div(part, TN));
    dim3 grid_scan(ceil_div(channels, SCAN_THREADS), n_seqs);
    LLMB_REQUIRE(grid_gates.y <= 65535 && grid_scan.y <= 65535, "gated_recurrence: too many tiles or sequences");
    float* u = work;
    float* decay = work + (size_t)n_tokens * channels;
    float* drive = decay + (size_t)n_tokens * channels;
    auto gates = long_step ? gates_kernel<8> : gates_kernel<2>;
#define LLMB_RECURRENCE(T)                                                                                          \
    do {                                                                                                            \
        ConvSource<T> source{(const T*)x, x_stride, state, conv_w, conv_b, taps, channels};                         \
        LLMB_CUDA(llmb::launch(conv_kernel<T>, dim3(n_tokens, ceil_div(channels, 256)), dim3(256), 0, stream, true, \
                               source, tok_seq, cu_seqlens, slot_ids, u));                                          \
        LLMB_CUDA(llmb::launch(gates, grid_gates, dim3(256), 0, stream, true, (const float*)u, channels, gate_a,    \
                               gate_a_bias, gate_i, gate_i_bias, part, rate, decay, drive, n_tokens));              \
        if (n_tokens == n_seqs && single_tokens) {                                                                  \
            LLMB_CUDA(llmb::launch(scan_single_kernel<T>, dim3(ceil_div(channels, 256), n_seqs), dim3(256), 0, stream, \
                                   true, (const T*)y, y_stride, (const T*)x, x_stride, (const float*)decay,         \
                                   (const float*)drive, state, taps, channels, slot_ids, (T*)out, out_stride,       \
                                   out_scale));                                                                     \
        } else if (n_tokens <= SCAN_SERIAL) {                                                                       \
            LLMB_CUDA(llmb::launch(scan_kernel<T>, grid_scan, dim3(SCAN_THREADS), 0, stream, true, (const T*)y,     \
                                   y_stride, (const T*)x, x_stride, (const float*)decay, (const float*)drive,       \
                                   state, taps, channels, cu_seqlens, slot_ids, (T*)out, out_stride, out_scale));   \
        } else {                                                                                                    \
            /* u is no longer needed: the chunks' products and end values take its place */                         \
            int n_chunks = ceil_div(n_tokens, SCAN_CHUNK);                                                          \
            float* products = u;                                                                                    \
            float* ends = u + (size_t)n_chunks * channels;                                                          \
            dim3 grid_chunks(ceil_div(channels, SCAN_THREADS), n_chunks);                                           \
            LLMB_REQUIRE(n_chunks <= 65535, "gated_recurrence: too many tokens in one call");                       \
            LLMB_CUDA(llmb::launch(scan_local_kernel, grid_chunks, dim3(SCAN_THREADS), 0, stream, true, decay,      \
                                   drive, (const float*)state, taps, channels, tok_seq, cu_seqlens, slot_ids,       \
                                   products, ends, n_tokens));                                                      \
            LLMB_CUDA(llmb::launch(scan_carry_kernel, dim3(ceil_div(channels, SCAN_THREADS)), dim3(SCAN_THREADS), 0, \
                                   stream, true, (const float*)products, ends, channels, n_chunks));                \
            LLMB_CUDA(llmb::launch(scan_apply_kernel<T>, grid_chunks, dim3(SCAN_THREADS), 0, stream, true,          \
                                   (const T*)y, y_stride, (const T*)x, x_stride, (const float*)decay,               \
                                   (const float*)drive, (const float*)ends, state, taps, channels, tok_seq,         \
                                   cu_seqlens, slot_ids, (T*)out, out_stride, out_scale, n_tokens));                \
        }                                                                                                           \
    } while (0)
    if (dtype == LLMB_DTYPE_F32) LLMB_RECURRENCE(float);
    else if (dtype == LLMB_DTYPE_BF16) LLMB_RECURRENCE(__nv_bfloat16);
    else return fail(LLMB_ERR_ARGUMENT, "gated_recurrence: unknown dtype %d", dtype);
#undef LLMB_RECURRENCE
    return check_launch("gated_recurrence");
}

LLMB_PACKED(llmb_gated_recurrence)
