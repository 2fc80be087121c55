// The selective scan of a Mamba mixer: per channel c a state of `states` numbers that decays by a step-dependent factor and takes
// the token's input along B, read along C:
//
//     step = softplus(pre[t, c])                      (pre = W_dt dt + bias, 32-bit)
//     S[c, n] <- exp(step * A[c, n]) S[c, n] + step * x[t, c] * B[t, n]          A = -exp(A_log)
//     y[t, c] = sum_n S[c, n] C[t, n] + D[c] x[t, c];        out[t, c] = y[t, c] * silu(z[t, c])
//
// A thread owns a channel of one sequence, keeps its states in registers and walks the run's tokens in order; B and C of a token
// are the same for every channel and are read through the cache as they are.  Everything is 32-bit; x and z arrive in the
// activations' dtype.  The state lives in the cache, [channels, states] floats per slot.  TAU_SCAN_STATES fixes `states`.
#include "common.cuh"

#ifndef TAU_SCAN_STATES
#error "compile with -DTAU_SCAN_STATES=<state numbers per channel>"
#endif

namespace {

constexpr int kStates = TAU_SCAN_STATES;
constexpr int kThreads = 64;

template <typename T>
__global__ void __launch_bounds__(kThreads)
selective_scan_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ z, long long z_stride, const float* __restrict__ pre,
                      const float* __restrict__ bc, const float* __restrict__ a_log, const float* __restrict__ skip, float* __restrict__ state,
                      const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, T* __restrict__ out, int channels) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int channel = blockIdx.x * kThreads + threadIdx.x, sequence = blockIdx.y;
    if (channel >= channels) return;
    float* record = state + (static_cast<size_t>(seq_slot[sequence]) * channels + channel) * kStates;
    float S[kStates], A[kStates];
#pragma unroll
    for (int n = 0; n < kStates; ++n) {
        S[n] = record[n];
        A[n] = -expf(a_log[static_cast<size_t>(channel) * kStates + n]);
    }
    const float d = skip[channel];
    const int begin = cu_seqlens[sequence], end = cu_seqlens[sequence + 1];
    for (int token = begin; token < end; ++token) {
        const float raw = pre[static_cast<size_t>(token) * channels + channel];
        const float step = raw > 20.0f ? raw : log1pf(expf(raw));
        const float input = to_float(x[static_cast<size_t>(token) * x_stride + channel]);
        const float gate = to_float(z[static_cast<size_t>(token) * z_stride + channel]);
        const float* b = bc + static_cast<size_t>(token) * 2 * kStates;
        const float* c = b + kStates;
        const float drive = step * input;
        float sums[2] = {0.0f, 0.0f};
#pragma unroll
        for (int n = 0; n < kStates; ++n) {
            S[n] = fmaf(expf(step * A[n]), S[n], drive * b[n]);
            sums[n & 1] = fmaf(S[n], c[n], sums[n & 1]);
        }
        const float y = fmaf(d, input, sums[0] + sums[1]);
        out[static_cast<size_t>(token) * channels + channel] = from_float<T>(y * gate / (1.0f + expf(-gate)));
    }
#pragma unroll
    for (int n = 0; n < kStates; ++n) record[n] = S[n];
}

}  // namespace

TAU_EXPORT int tau_scan_states() { return kStates; }

// x, z [tokens, channels] with their own row strides; pre [tokens, channels]; bc [tokens, 2 * states] (B, then C); a_log [channels, states];
// skip [channels]; state [slots, channels * states]; out [tokens, channels] contiguous.
TAU_EXPORT int tau_selective_scan(int dtype, const void* x, long long x_stride, const void* z, long long z_stride, const float* pre, const float* bc,
                                  const float* a_log, const float* skip, float* state, const int* cu_seqlens, const int* seq_slot, void* out, int n_seqs,
                                  int channels, void* stream) {
    if (n_seqs <= 0) return 0;
    if (!x || !z || !pre || !bc || !a_log || !skip || !state || !cu_seqlens || !seq_slot || !out || channels <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    dim3 grid((channels + kThreads - 1) / kThreads, n_seqs), block(kThreads);
    if (dtype == TAU_F32)
        tau_launch(selective_scan_kernel<float>, grid, block, 0, s, static_cast<const float*>(x), x_stride, static_cast<const float*>(z), z_stride, pre, bc,
                   a_log, skip, state, cu_seqlens, seq_slot, static_cast<float*>(out), channels);
    else if (dtype == TAU_BF16)
        tau_launch(selective_scan_kernel<bf16>, grid, block, 0, s, static_cast<const bf16*>(x), x_stride, static_cast<const bf16*>(z), z_stride, pre, bc,
                   a_log, skip, state, cu_seqlens, seq_slot, static_cast<bf16*>(out), channels);
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}
