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
// Two kernels. conv_gates: tiles of 32 tokens x 64 channels of one part; the u values of the tile's
// tokens are formed on the fly from x and the state (a value is `taps` multiply-adds), both gates
// share them; it writes a and the driving term sqrt(1 - a^2) i u of every token. scan: one thread per
// (sequence, channel) walks the sequence's tokens of this step in order, then brings the state up to
// date (S, and the last taps - 1 inputs). The first kernel only reads the state, the second writes it.
#include "common.cuh"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_gated_recurrence)

constexpr int MAX_TAPS = 16;
constexpr int TM = 32;        // tokens of a tile
constexpr int TN = 64;        // output channels of a tile
constexpr int KC = 32;        // input channels staged at a time

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
conv_gates_kernel(ConvSource<T> source, const float* __restrict__ gate_a, const float* __restrict__ gate_a_bias,
                  const float* __restrict__ gate_i, const float* __restrict__ gate_i_bias, int part,
                  const float* __restrict__ rate, const int* __restrict__ tok_seq, const int* __restrict__ cu_seqlens,
                  const int* __restrict__ slot_ids, float* __restrict__ decay, float* __restrict__ drive, int n_tokens) {
    __shared__ float u_tile[TM][KC + 1];
    __shared__ float a_tile[TN][KC + 1];
    __shared__ float i_tile[TN][KC + 1];
    __shared__ int start_of[TM], slot_of[TM];
    griddep_launch();
    griddep_wait();
    int channels = source.channels;
    int tiles_per_part = (part + TN - 1) / TN;
    int b = blockIdx.y / tiles_per_part;                 // which part of the channels
    int o0 = (blockIdx.y % tiles_per_part) * TN;         // first output of the tile, inside the part
    int t0 = blockIdx.x * TM;
    if (threadIdx.x < TM) {
        int t = t0 + threadIdx.x;
        int seq = t < n_tokens ? tok_seq[t] : 0;
        start_of[threadIdx.x] = t < n_tokens ? cu_seqlens[seq] : 0;
        slot_of[threadIdx.x] = t < n_tokens ? slot_ids[seq] : 0;
    }
    __syncthreads();
    // thread (ty, tx) owns tokens ty, ty + 8, ty + 16, ty + 24 and outputs tx, tx + 32
    int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    float acc_a[4][2], acc_i[4][2];
#pragma unroll
    for (int m = 0; m < 4; ++m)
#pragma unroll
        for (int n = 0; n < 2; ++n) acc_a[m][n] = acc_i[m][n] = 0.f;
    const float* wa = gate_a + (size_t)b * part * part;
    const float* wi = gate_i + (size_t)b * part * part;
    for (int k0 = 0; k0 < part; k0 += KC) {
        for (int e = threadIdx.x; e < TM * KC; e += 256) {
            int m = e / KC, k = e % KC;
            int t = t0 + m;
            u_tile[m][k] = (t < n_tokens && k0 + k < part)
                               ? source.value(t, start_of[m], slot_of[m], b * part + k0 + k) : 0.f;
        }
        for (int e = threadIdx.x; e < TN * KC; e += 256) {
            int n = e / KC, k = e % KC;
            bool live = o0 + n < part && k0 + k < part;
            size_t at = (size_t)(o0 + n) * part + k0 + k;
            a_tile[n][k] = live ? wa[at] : 0.f;
            i_tile[n][k] = live ? wi[at] : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < KC; ++k) {
            float un[4], an[2], in[2];
#pragma unroll
            for (int m = 0; m < 4; ++m) un[m] = u_tile[ty + 8 * m][k];
#pragma unroll
            for (int n = 0; n < 2; ++n) { an[n] = a_tile[tx + 32 * n][k]; in[n] = i_tile[tx + 32 * n][k]; }
#pragma unroll
            for (int m = 0; m < 4; ++m)
#pragma unroll
                for (int n = 0; n < 2; ++n) {
                    acc_a[m][n] = fmaf(an[n], un[m], acc_a[m][n]);
                    acc_i[m][n] = fmaf(in[n], un[m], acc_i[m][n]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        int t = t0 + ty + 8 * m;
        if (t >= n_tokens) continue;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            int o = o0 + tx + 32 * n;
            if (o >= part) continue;
            int c = b * part + o;
            float u = source.value(t, start_of[ty + 8 * m], slot_of[ty + 8 * m], c);
            float r = 1.0f / (1.0f + expf(-(acc_a[m][n] + gate_a_bias[c])));
            float g = 1.0f / (1.0f + expf(-(acc_i[m][n] + gate_i_bias[c])));
            float a = expf(rate[c] * r);
            decay[(size_t)t * channels + c] = a;
            drive[(size_t)t * channels + c] = sqrtf(1.0f - a * a) * g * u;
        }
    }
}

__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void __launch_bounds__(128)
scan_kernel(const T* __restrict__ y, int y_stride, const T* __restrict__ x, int x_stride,
            const float* __restrict__ decay, const float* __restrict__ drive, float* __restrict__ state, int taps,
            int channels, const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids, T* __restrict__ out,
            int out_stride, float out_scale) {
    griddep_launch();
    griddep_wait();
    int c = blockIdx.x * 128 + threadIdx.x;
    if (c >= channels) return;
    int seq = blockIdx.y;
    int first = cu_seqlens[seq], last = cu_seqlens[seq + 1];
    if (first >= last) return;
    float* rows = state + (size_t)slot_ids[seq] * taps * channels + c;      // row r at rows[r * channels]
    float s = rows[(size_t)(taps - 1) * channels];
#pragma unroll 4
    for (int t = first; t < last; ++t) {
        s = fmaf(decay[(size_t)t * channels + c], s, drive[(size_t)t * channels + c]);
        out[(size_t)t * out_stride + c] = from_float<T>(s * gelu_tanh(to_float(y[(size_t)t * y_stride + c])) * out_scale);
    }
    rows[(size_t)(taps - 1) * channels] = s;
    // the last taps - 1 inputs: row r of the new state is input (count - (taps - 1) + r) of this step, or, where
    // that lies before the step, row (r + count) of the old state
    int count = last - first;
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

// work [2, T, C] float32: a, then the driving term.
LLMB_EXPORT int llmb_gated_recurrence(const void* y, int y_stride, const void* x, int x_stride, int dtype,
                                      const float* conv_w, const float* conv_b, int taps, const float* gate_a,
                                      const float* gate_a_bias, const float* gate_i, const float* gate_i_bias,
                                      int blocks, const float* rate, float* state, const int* tok_seq,
                                      const int* cu_seqlens, const int* slot_ids, void* out, int out_stride,
                                      float out_scale, float* work, int n_tokens, int channels, int n_seqs,
                                      cudaStream_t stream) {
    if (n_tokens == 0) return LLMB_OK;
    LLMB_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "gated_recurrence: %d taps (1 to %d are built)", taps, MAX_TAPS);
    LLMB_REQUIRE(channels > 0 && blocks > 0 && channels % blocks == 0 && n_seqs > 0,
                 "gated_recurrence: %d channels in %d parts", channels, blocks);
    int part = channels / blocks;
    dim3 grid_gates(ceil_div(n_tokens, TM), blocks * ceil_div(part, TN));
    dim3 grid_scan(ceil_div(channels, 128), n_seqs);
    LLMB_REQUIRE(grid_gates.y <= 65535 && grid_scan.y <= 65535, "gated_recurrence: too many tiles or sequences");
    float* decay = work;
    float* drive = work + (size_t)n_tokens * channels;
#define LLMB_RECURRENCE(T)                                                                                          \
    do {                                                                                                            \
        ConvSource<T> source{(const T*)x, x_stride, state, conv_w, conv_b, taps, channels};                         \
        LLMB_CUDA(llmb::launch(conv_gates_kernel<T>, grid_gates, dim3(256), 0, stream, true, source, gate_a,        \
                               gate_a_bias, gate_i, gate_i_bias, part, rate, tok_seq, cu_seqlens, slot_ids, decay,  \
                               drive, n_tokens));                                                                   \
        LLMB_CUDA(llmb::launch(scan_kernel<T>, grid_scan, dim3(128), 0, stream, true, (const T*)y, y_stride,        \
                               (const T*)x, x_stride, (const float*)decay, (const float*)drive, state, taps,        \
                               channels, cu_seqlens, slot_ids, (T*)out, out_stride, out_scale));                    \
    } while (0)
    if (dtype == LLMB_DTYPE_F32) LLMB_RECURRENCE(float);
    else if (dtype == LLMB_DTYPE_BF16) LLMB_RECURRENCE(__nv_bfloat16);
    else return fail(LLMB_ERR_ARGUMENT, "gated_recurrence: unknown dtype %d", dtype);
#undef LLMB_RECURRENCE
    return check_launch("gated_recurrence");
}

LLMB_PACKED(llmb_gated_recurrence)
