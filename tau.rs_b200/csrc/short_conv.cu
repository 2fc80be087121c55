// A short causal convolution over time on each channel of a projection, with the sequence's last inputs carried as state:
//
//     out[t, c] = act(bias[c] + sum_j w[j, c] * x[t - (taps - 1) + j, c])        j = 0 .. taps - 1, the last tap weighs the token itself
//
// Rows before a sequence's run of new tokens come from state[slot] ([taps - 1, channels], 32-bit, oldest first; zeros when the
// sequence starts); afterwards the state becomes the last taps - 1 inputs again.  The weights arrive tap by tap ([taps, channels]),
// so that a tap's channels lie side by side.  Sums are 32-bit; the activation is SiLU or none.  A step of single tokens moves the
// state on in the same launch, a step with longer runs in a second launch over (sequence, block of channels).
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

template <typename T, typename O>
__global__ void __launch_bounds__(kThreads)
short_conv_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ weight, const float* __restrict__ bias, float* __restrict__ state,
                  const int* __restrict__ token_seq, const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, O* __restrict__ out,
                  long long out_stride, int channels, int taps, int silu, int move_state) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int token = blockIdx.x, channel = blockIdx.y * kThreads + threadIdx.x;
    if (channel >= channels) return;
    const int sequence = token_seq[token], begin = cu_seqlens[sequence];
    float* record = taps > 1 ? state + static_cast<size_t>(seq_slot[sequence]) * (taps - 1) * channels : nullptr;
    float sum = bias ? bias[channel] : 0.0f;
    for (int tap = 0; tap < taps; ++tap) {
        const int source = token - (taps - 1 - tap);
        // `begin - source` rows before the run: the state's row (taps - 1) - (begin - source).
        const float value = source >= begin ? to_float(x[static_cast<size_t>(source) * x_stride + channel])
                                            : record[static_cast<size_t>(taps - 1 - (begin - source)) * channels + channel];
        sum = fmaf(weight[static_cast<size_t>(tap) * channels + channel], value, sum);
    }
    if (move_state && taps > 1) {       // one token per sequence: this thread alone reads and writes its channel of the record
        for (int row = 0; row + 2 < taps; ++row) record[static_cast<size_t>(row) * channels + channel] = record[static_cast<size_t>(row + 1) * channels + channel];
        record[static_cast<size_t>(taps - 2) * channels + channel] = to_float(x[static_cast<size_t>(token) * x_stride + channel]);
    }
    if (silu) sum = sum / (1.0f + expf(-sum));
    out[static_cast<size_t>(token) * out_stride + channel] = from_float<O>(sum);
}

// grid (sequences, blocks of channels): the record becomes the last taps - 1 of (record, the run's inputs).
template <typename T>
__global__ void __launch_bounds__(kThreads)
short_conv_state_kernel(const T* __restrict__ x, long long x_stride, float* __restrict__ state, const int* __restrict__ cu_seqlens,
                        const int* __restrict__ seq_slot, int channels, int taps) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int sequence = blockIdx.x, channel = blockIdx.y * kThreads + threadIdx.x;
    if (channel >= channels) return;
    const int begin = cu_seqlens[sequence], end = cu_seqlens[sequence + 1], count = end - begin;
    float* record = state + static_cast<size_t>(seq_slot[sequence]) * (taps - 1) * channels;
    for (int row = 0; row < taps - 1; ++row) {     // rising rows read what lies behind them, so the record is renewed in place
        const int old = row + count;
        record[static_cast<size_t>(row) * channels + channel] =
            old < taps - 1 ? record[static_cast<size_t>(old) * channels + channel]
                           : to_float(x[static_cast<size_t>(end - (taps - 1 - row)) * x_stride + channel]);
    }
}

template <typename T, typename O>
int launch(const void* x, long long x_stride, const float* weight, const float* bias, float* state, const int* token_seq, const int* cu_seqlens,
           const int* seq_slot, void* out, long long out_stride, int tokens, int n_seqs, int channels, int taps, int silu, int update, int single,
           cudaStream_t s) {
    const int blocks = (channels + kThreads - 1) / kThreads;
    tau_launch(short_conv_kernel<T, O>, dim3(tokens, blocks), dim3(kThreads), 0, s, static_cast<const T*>(x), x_stride, weight, bias, state, token_seq,
               cu_seqlens, seq_slot, static_cast<O*>(out), out_stride, channels, taps, silu, (update && single) ? 1 : 0);
    int status = tau_launch_status();
    if (status != 0 || !update || single || taps <= 1) return status;
    tau_launch(short_conv_state_kernel<T>, dim3(n_seqs, blocks), dim3(kThreads), 0, s, static_cast<const T*>(x), x_stride, state, cu_seqlens, seq_slot,
               channels, taps);
    return tau_launch_status();
}

}  // namespace

// x [tokens, >= channels] rows `x_stride` apart; out rows `out_stride` apart, of dtype `out_dtype`.
TAU_EXPORT int tau_short_conv(int dtype, int out_dtype, const void* x, long long x_stride, const float* weight, const float* bias, float* state,
                              const int* token_seq, const int* cu_seqlens, const int* seq_slot, void* out, long long out_stride, int tokens, int n_seqs,
                              int channels, int taps, int silu, int update, int single, void* stream) {
    if (tokens <= 0) return 0;
    if (!x || !weight || !out || !token_seq || !cu_seqlens || !seq_slot || channels <= 0 || taps <= 0 || (taps > 1 && !state)) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define TAU_CONV(T, O) return launch<T, O>(x, x_stride, weight, bias, state, token_seq, cu_seqlens, seq_slot, out, out_stride, tokens, n_seqs, channels, taps, silu, update, single, s)
    if (dtype == TAU_F32 && out_dtype == TAU_F32) TAU_CONV(float, float);
    if (dtype == TAU_BF16 && out_dtype == TAU_F32) TAU_CONV(bf16, float);
    if (dtype == TAU_BF16 && out_dtype == TAU_BF16) TAU_CONV(bf16, bf16);
#undef TAU_CONV
    return cudaErrorInvalidValue;
}
