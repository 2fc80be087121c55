// The selective scan of a Mamba mixer: per channel c a state of `states` numbers that decays by a step-dependent factor and takes
// the token's input along B, read along C:
//
//     step = softplus(pre[t, c])                      (pre = W_dt dt + bias, 32-bit)
//     S[c, n] <- exp(step * A[c, n]) S[c, n] + step * x[t, c] * B[t, n]          A = -exp(A_log)
//     y[t, c] = sum_n S[c, n] C[t, n] + D[c] x[t, c];        out[t, c] = y[t, c] * silu(z[t, c])
//
// Single tokens: a thread owns a channel of one sequence, keeps its states in registers and walks the run's tokens in order; B and C
// of a token are the same for every channel and are read through the cache as they are.
// Runs of tokens: a block of four warps owns a tile of channels of one sequence.  Two warps stage the next tile of tokens in shared
// memory, all their loads in flight at once, and do there what does not depend on the state (softplus, step * x, silu(z)); the other
// two walk the tile that was staged before, kSplit threads to a channel with states / kSplit state numbers each in registers, so
// that a token costs a few dependent instructions instead of a round trip to memory.  One barrier per tile.
// Everything is 32-bit; x and z arrive in the activations' dtype.  The state lives in the cache, [channels, states] floats per slot.
// TAU_SCAN_STATES fixes `states`.
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

constexpr int kSplit = kStates % 4 == 0 ? 4 : kStates % 2 == 0 ? 2 : 1;   // threads that share a channel
constexpr int kPer = kStates / kSplit;                                      // state numbers of a thread
constexpr int kWalkers = 64;                                                // walking threads, and as many staging ones
constexpr int kTileChannels = kWalkers / kSplit;
constexpr int kWide = kStates <= 32 ? 64 : kStates <= 64 ? 32 : 16;
constexpr int kTile = kWide < 16 * kSplit ? kWide : 16 * kSplit;              // tokens staged at once: at most 16 pairs to a staging thread
constexpr int kEach = kTile * kTileChannels / kWalkers;                     // (token, channel) pairs that a staging thread prepares
constexpr int kPlane = kTile * kTileChannels;                               // step | step * x | x | silu(z) planes, then B and C
constexpr int kBufferFloats = 4 * kPlane + kTile * 2 * kStates;
constexpr int kTiledBytes = 2 * kBufferFloats * 4;

// grid: (ceil(channels / kTileChannels), sequences); block: 2 * kWalkers.  Dynamic shared memory: kTiledBytes.
template <typename T>
__global__ void __launch_bounds__(2 * kWalkers)
selective_scan_tiled_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ z, long long z_stride, const float* __restrict__ pre,
                            const float* __restrict__ bc, const float* __restrict__ a_log, const float* __restrict__ skip, float* __restrict__ state,
                            const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, T* __restrict__ out, int channels) {
    grid_dependents_launch();
    grid_dependency_wait();
    extern __shared__ __align__(16) float staged[];
    const int sequence = blockIdx.y, channel0 = blockIdx.x * kTileChannels;
    const int begin = cu_seqlens[sequence], end = cu_seqlens[sequence + 1];
    const int n_tiles = (end - begin + kTile - 1) / kTile;
    const bool walker = threadIdx.x < kWalkers;
    const int lane_id = walker ? threadIdx.x : threadIdx.x - kWalkers;
    // walkers: channel and part of its states; stagers: channel and first token of the tile
    const int local = walker ? lane_id / kSplit : lane_id % kTileChannels;
    const int part = walker ? lane_id % kSplit : lane_id / kTileChannels;
    const bool real = channel0 + local < channels;
    const int channel = real ? channel0 + local : channels - 1;
    float S[kPer], A[kPer];
    float* record = state + (static_cast<size_t>(seq_slot[sequence]) * channels + channel) * kStates + part * kPer;
    if (walker) {
#pragma unroll
        for (int r = 0; r < kPer; ++r) {
            S[r] = record[r];
            A[r] = -expf(a_log[static_cast<size_t>(channel) * kStates + part * kPer + r]);
        }
    }
    const float d = skip[channel];

    auto stage = [&](int tile) {
        float* buffer = staged + (tile & 1) * kBufferFloats;
        const int token0 = begin + tile * kTile;
        const int count = end - token0 < kTile ? end - token0 : kTile;
        float raw[kEach], input[kEach], gate[kEach];
#pragma unroll
        for (int e = 0; e < kEach; ++e) {
            const int i = part + e * kSplit;
            const size_t token = static_cast<size_t>(token0 + (i < count ? i : 0));
            raw[e] = pre[token * channels + channel];
            input[e] = to_float(x[token * x_stride + channel]);
            gate[e] = to_float(z[token * z_stride + channel]);
        }
        const float* source = bc + static_cast<size_t>(token0) * 2 * kStates;
        float* target = buffer + 4 * kPlane;
        if constexpr (kStates % 2 == 0) {      // rows of B and C are multiples of 16 bytes
            const float4* source4 = reinterpret_cast<const float4*>(source);
            float4* target4 = reinterpret_cast<float4*>(target);
#pragma unroll 4
            for (int j = lane_id; j < count * (kStates / 2); j += kWalkers) target4[j] = source4[j];
        } else {
#pragma unroll 4
            for (int j = lane_id; j < count * 2 * kStates; j += kWalkers) target[j] = source[j];
        }
#pragma unroll
        for (int e = 0; e < kEach; ++e) {
            const int at = (part + e * kSplit) * kTileChannels + local;
            const float step = raw[e] > 20.0f ? raw[e] : log1pf(expf(raw[e]));
            buffer[at] = step;
            buffer[kPlane + at] = step * input[e];
            buffer[2 * kPlane + at] = input[e];
            buffer[3 * kPlane + at] = gate[e] / (1.0f + expf(-gate[e]));
        }
    };

    if (!walker && n_tiles > 0) stage(0);
    __syncthreads();
    for (int tile = 0; tile < n_tiles; ++tile) {
        if (!walker) {
            if (tile + 1 < n_tiles) stage(tile + 1);
        } else {
            const float* buffer = staged + (tile & 1) * kBufferFloats;
            const int token0 = begin + tile * kTile;
            const int count = end - token0 < kTile ? end - token0 : kTile;
            // Four tokens to a round: only the state's own multiply-add waits for the token before, the rest of the tokens overlap.
#pragma unroll 4
            for (int i = 0; i < count; ++i) {
                const int at = i * kTileChannels + local;
                const float step = buffer[at], drive = buffer[kPlane + at];
                const float* b = buffer + 4 * kPlane + i * 2 * kStates + part * kPer;
                const float* c = b + kStates;
                float sums[2] = {0.0f, 0.0f};
#pragma unroll
                for (int r = 0; r < kPer; ++r) {
                    S[r] = fmaf(expf(step * A[r]), S[r], drive * b[r]);
                    sums[r & 1] = fmaf(S[r], c[r], sums[r & 1]);
                }
                float sum = sums[0] + sums[1];
#pragma unroll
                for (int m = 1; m < kSplit; m <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
                if (part == 0 && real)
                    out[static_cast<size_t>(token0 + i) * channels + channel] = from_float<T>(fmaf(d, buffer[2 * kPlane + at], sum) * buffer[3 * kPlane + at]);
            }
        }
        __syncthreads();      // the tile that was walked may be written over; the tile that was staged may be walked
    }
    if (walker && real) {
#pragma unroll
        for (int r = 0; r < kPer; ++r) record[r] = S[r];
    }
}

template <typename T>
int launch_tiled(const void* x, long long x_stride, const void* z, long long z_stride, const float* pre, const float* bc, const float* a_log,
                 const float* skip, float* state, const int* cu_seqlens, const int* seq_slot, void* out, int n_seqs, int channels, cudaStream_t s) {
    static bool configured = false;
    if (!configured && kTiledBytes > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(selective_scan_tiled_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTiledBytes);
        if (status != cudaSuccess) return static_cast<int>(status);
    }
    configured = true;
    dim3 grid((channels + kTileChannels - 1) / kTileChannels, n_seqs), block(2 * kWalkers);
    tau_launch(selective_scan_tiled_kernel<T>, grid, block, kTiledBytes, s, static_cast<const T*>(x), x_stride, static_cast<const T*>(z), z_stride, pre, bc,
               a_log, skip, state, cu_seqlens, seq_slot, static_cast<T*>(out), channels);
    return tau_launch_status();
}

}  // namespace

TAU_EXPORT int tau_scan_states() { return kStates; }

// x, z [tokens, channels] with their own row strides; pre [tokens, channels]; bc [tokens, 2 * states] (B, then C); a_log [channels, states];
// skip [channels]; state [slots, channels * states]; out [tokens, channels] contiguous.  `tokens` > `n_seqs` (some run is longer than
// one token) takes the tiled kernel.
TAU_EXPORT int tau_selective_scan(int dtype, const void* x, long long x_stride, const void* z, long long z_stride, const float* pre, const float* bc,
                                  const float* a_log, const float* skip, float* state, const int* cu_seqlens, const int* seq_slot, void* out, int n_seqs,
                                  int tokens, int channels, void* stream) {
    if (n_seqs <= 0 || tokens <= 0) return 0;
    if (!x || !z || !pre || !bc || !a_log || !skip || !state || !cu_seqlens || !seq_slot || !out || channels <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (tokens > n_seqs) {
        if (dtype == TAU_F32) return launch_tiled<float>(x, x_stride, z, z_stride, pre, bc, a_log, skip, state, cu_seqlens, seq_slot, out, n_seqs, channels, s);
        if (dtype == TAU_BF16) return launch_tiled<bf16>(x, x_stride, z, z_stride, pre, bc, a_log, skip, state, cu_seqlens, seq_slot, out, n_seqs, channels, s);
        return cudaErrorInvalidValue;
    }
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
