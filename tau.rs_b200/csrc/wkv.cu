// A matrix state per head with a decay per key channel and a bonus for the token itself (time mixing in the manner of RWKV):
//
//     o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t            S_t = diag(w_t) S_(t-1) + k_t v_t^T            (S is key_dim x value_dim)
//
// so the read-out sees the states of the tokens before and the token's own k v^T weighed by the head's bonus u; the state then decays
// by w_t per key channel and takes k v^T unweighed.
//
//   shift:   every projection reads its own mix of the token's input h and the input of the token before (h' = the sequence's kept
//            last input for a run's first token, zeros when the sequence starts): mix_s = h + (h' - h) * mu_s, for `mixes` vectors mu.
//   decay:   in place, w = exp(-exp(x + w0)) per head and key channel; and tanh in place for the low-rank step before it.
//   walk:    one block owns (sequence, head, tile of value columns) and walks the run's tokens in order, the next tokens' r, k, w and
//            values on their way into shared memory meanwhile (cp.async).  A column of S is shared by kSplit threads with kRows key
//            rows each in registers; a token costs one pass over the rows, and the threads of a column meet once in four tokens (two for very wide keys).
//
// The state is 32-bit and lives in the cache, [heads, value_dim, key_dim] per slot.  TAU_KEY_DIM fixes key_dim.
#include "common.cuh"

#ifndef TAU_KEY_DIM
#error "compile with -DTAU_KEY_DIM=<key elements per head>"
#endif

namespace {

constexpr int kDim = TAU_KEY_DIM;
// Threads that share a column: four key rows to a thread where the width allows, so that a token's chain of dependent instructions is
// short and a scheduler has warps to choose from even when a prompt brings one block to an SM.
constexpr int kSplit = kDim <= 4 ? 1 : kDim <= 8 ? 2 : kDim <= 16 ? 4 : kDim <= 32 ? 8 : kDim <= 64 ? 16 : 32;
constexpr int kRows = (kDim + kSplit - 1) / kSplit;
constexpr bool kExact = kDim % kSplit == 0;
constexpr int kThreads = 256;

// grid (tokens, blocks of columns).  x [tokens, width]; last [slots, width] float: each sequence's last input.  mu [mixes, width];
// out [mixes, tokens, width].  With `move` (every sequence brings one token) the thread that read the kept input replaces it.
template <typename T>
__global__ void __launch_bounds__(kThreads)
token_shift_kernel(const T* __restrict__ x, const float* __restrict__ mu, float* __restrict__ last, const int* __restrict__ token_seq,
                   const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, T* __restrict__ out, int tokens, int width, int mixes, int move) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int token = blockIdx.x, column = blockIdx.y * kThreads + threadIdx.x;
    if (column >= width) return;
    const int sequence = token_seq[token];
    const float here = to_float(x[static_cast<size_t>(token) * width + column]);
    float* kept = last + static_cast<size_t>(seq_slot[sequence]) * width + column;
    const float before = token > cu_seqlens[sequence] ? to_float(x[static_cast<size_t>(token - 1) * width + column]) : *kept;
    for (int mix = 0; mix < mixes; ++mix)
        out[(static_cast<size_t>(mix) * tokens + token) * width + column] = from_float<T>(fmaf(before - here, mu[static_cast<size_t>(mix) * width + column], here));
    if (move) *kept = here;
}

// grid (sequences, blocks of columns): the kept input becomes the run's last.
template <typename T>
__global__ void __launch_bounds__(kThreads)
token_shift_keep_kernel(const T* __restrict__ x, float* __restrict__ last, const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, int width) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int sequence = blockIdx.x, column = blockIdx.y * kThreads + threadIdx.x;
    if (column >= width) return;
    const int end = cu_seqlens[sequence + 1];
    if (end > cu_seqlens[sequence]) last[static_cast<size_t>(seq_slot[sequence]) * width + column] = to_float(x[static_cast<size_t>(end - 1) * width + column]);
}

template <typename T>
__global__ void tanh_kernel(T* __restrict__ values, long long count) {
    grid_dependents_launch();
    grid_dependency_wait();
    for (long long index = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; index < count; index += static_cast<long long>(gridDim.x) * blockDim.x)
        values[index] = from_float<T>(tanhf(to_float(values[index])));
}

__global__ void channel_decay_kernel(float* __restrict__ values, const float* __restrict__ offset, long long count, int width) {
    grid_dependents_launch();
    grid_dependency_wait();
    for (long long index = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; index < count; index += static_cast<long long>(gridDim.x) * blockDim.x)
        values[index] = expf(-expf(values[index] + offset[index % width]));
}

__device__ __forceinline__ void copy_float(float* target, const float* source) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(target))), "l"(source) : "memory");
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// r, k, w [tokens, heads * kDim], v [tokens, heads * value_dim], bonus [heads, kDim], all float; out [tokens, heads * value_dim] float.
// A thread's rows of S depend on nobody else's, so the walk takes kGroup tokens between two barriers: the threads that share a column
// meet only to add up their parts of the read-outs, once per group, and a group's r, k, w and values arrive as one set of copies while
// the groups before are walked (kDepth groups in the ring: a set of copies has kDepth - 1 groups' time to arrive).
constexpr int kGroup = kDim <= 256 ? 4 : 2;      // (two for very wide keys: the ring stays within the static shared memory)

constexpr int kDepth = kDim <= 64 ? 4 : kDim <= 128 ? 3 : 2;

template <int kColumns>
__global__ void __launch_bounds__(kColumns * kSplit)
wkv_kernel(const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ w, const float* __restrict__ bonus,
           float* __restrict__ state, long long slot_stride, const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, float* __restrict__ out,
           int heads, int value_dim) {
    grid_dependents_launch();
    grid_dependency_wait();
    __shared__ __align__(16) float rs[kDepth][kGroup][kDim], ks[kDepth][kGroup][kDim], ws[kDepth][kGroup][kDim];
    __shared__ float vs[kDepth][kGroup][kColumns], parts[kGroup][kSplit][kColumns];
    const int head = blockIdx.x, sequence = blockIdx.y;
    const int local = threadIdx.x % kColumns, part = threadIdx.x / kColumns, row0 = part * kRows;
    const int column = blockIdx.z * kColumns + local;
    const bool live = column < value_dim;
    float* record = state + static_cast<size_t>(seq_slot[sequence]) * slot_stride + (static_cast<size_t>(head) * value_dim + (live ? column : 0)) * kDim;
    float S[kRows], own[kRows];
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
        S[i] = (live && row0 + i < kDim) ? record[row0 + i] : 0.0f;
        own[i] = row0 + i < kDim ? bonus[static_cast<size_t>(head) * kDim + row0 + i] : 0.0f;
    }
    const int begin = cu_seqlens[sequence], end = cu_seqlens[sequence + 1];
    const int groups = (end - begin + kGroup - 1) / kGroup;
    constexpr int kStage = (kDim + kColumns * kSplit - 1) / (kColumns * kSplit);
    // One set of copies per group of tokens, empty ones too, so that the count of sets in flight says which groups have arrived.
    auto stage = [&](int group) {
        const int half = group % kDepth;
#pragma unroll
        for (int t = 0; t < kGroup; ++t) {
            const int token = begin + group * kGroup + t;
            if (group < groups && token < end) {
                const size_t keys = (static_cast<size_t>(token) * heads + head) * kDim;
#pragma unroll
                for (int i = 0; i < kStage; ++i) {
                    const int d = threadIdx.x + i * kColumns * kSplit;
                    if (d < kDim) {
                        copy_float(&rs[half][t][d], r + keys + d);
                        copy_float(&ks[half][t][d], k + keys + d);
                        copy_float(&ws[half][t][d], w + keys + d);
                    }
                }
                if (part == 0 && live) copy_float(&vs[half][t][local], v + (static_cast<size_t>(token) * heads + head) * value_dim + column);
            }
        }
        copy_commit();
    };
#pragma unroll
    for (int group = 0; group < kDepth; ++group) stage(group);
    for (int group = 0; group < groups; ++group) {
        const int half = group % kDepth, first = begin + group * kGroup;
        const int count = end - first < kGroup ? end - first : kGroup;
        copy_wait<kDepth - 1>();      // this thread's copies of the group are done (those of the next groups may be on their way)
        __syncthreads();     // everybody's are; and the parts of the group before have been added up
        // A whole group is walked without a branch, so that the loads of all its tokens can be on their way at once.
        auto walk = [&](int t) {
            const float value = live ? vs[half][t][local] : 0.0f;
            float sums[2] = {0.0f, 0.0f};
#pragma unroll
            for (int i = 0; i < kRows; ++i) {
                if (kExact || row0 + i < kDim) {
                    const float write = ks[half][t][row0 + i] * value;                 // the token's own k v^T, this thread's rows of this column
                    sums[i & 1] = fmaf(fmaf(own[i], write, S[i]), rs[half][t][row0 + i], sums[i & 1]);
                    S[i] = fmaf(ws[half][t][row0 + i], S[i], write);
                }
            }
            parts[t][part][local] = sums[0] + sums[1];
        };
        if (count == kGroup) {
#pragma unroll
            for (int t = 0; t < kGroup; ++t) walk(t);
        } else {
            for (int t = 0; t < count; ++t) walk(t);
        }
        __syncthreads();     // the parts are complete, and the group's place in the ring may be written over
        stage(group + kDepth);
        if (live) {      // the threads of a column share the group's tokens among them
            for (int t = part; t < count; t += kSplit) {
                float sum = 0.0f;
#pragma unroll
                for (int p = 0; p < kSplit; ++p) sum += parts[t][p][local];
                out[(static_cast<size_t>(first + t) * heads + head) * value_dim + column] = sum;
            }
        }
    }
    copy_wait<0>();
    if (live) {
#pragma unroll
        for (int i = 0; i < kRows; ++i)
            if (row0 + i < kDim) record[row0 + i] = S[i];
    }
}

}  // namespace

TAU_EXPORT int tau_wkv_key_dim() { return kDim; }

// x [tokens, width] of `dtype`; out [mixes, tokens, width] of the same; last [slots, width] float.  `update`: the kept inputs move on
// (in the same launch where `single` says that every sequence brings one token, else in a second one).
TAU_EXPORT int tau_token_shift(int dtype, const void* x, const float* mu, float* last, const int* token_seq, const int* cu_seqlens, const int* seq_slot,
                               void* out, int tokens, int n_seqs, int width, int mixes, int update, int single, void* stream) {
    if (tokens <= 0) return 0;
    if (!x || !mu || !last || !token_seq || !cu_seqlens || !seq_slot || !out || width <= 0 || mixes <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int blocks = (width + kThreads - 1) / kThreads;
    const int move = (update && single) ? 1 : 0;
    if (dtype == TAU_F32)
        tau_launch(token_shift_kernel<float>, dim3(tokens, blocks), dim3(kThreads), 0, s, static_cast<const float*>(x), mu, last, token_seq, cu_seqlens, seq_slot,
                   static_cast<float*>(out), tokens, width, mixes, move);
    else if (dtype == TAU_BF16)
        tau_launch(token_shift_kernel<bf16>, dim3(tokens, blocks), dim3(kThreads), 0, s, static_cast<const bf16*>(x), mu, last, token_seq, cu_seqlens, seq_slot,
                   static_cast<bf16*>(out), tokens, width, mixes, move);
    else return cudaErrorInvalidValue;
    int status = tau_launch_status();
    if (status != 0 || !update || single) return status;
    if (dtype == TAU_F32) tau_launch(token_shift_keep_kernel<float>, dim3(n_seqs, blocks), dim3(kThreads), 0, s, static_cast<const float*>(x), last, cu_seqlens, seq_slot, width);
    else tau_launch(token_shift_keep_kernel<bf16>, dim3(n_seqs, blocks), dim3(kThreads), 0, s, static_cast<const bf16*>(x), last, cu_seqlens, seq_slot, width);
    return tau_launch_status();
}

TAU_EXPORT int tau_tanh(int dtype, void* values, long long count, void* stream) {
    if (count <= 0) return 0;
    if (!values) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned blocks = static_cast<unsigned>((count + 255) / 256 < 1184 ? (count + 255) / 256 : 1184);
    if (dtype == TAU_F32) tau_launch(tanh_kernel<float>, dim3(blocks), dim3(256), 0, s, static_cast<float*>(values), count);
    else if (dtype == TAU_BF16) tau_launch(tanh_kernel<bf16>, dim3(blocks), dim3(256), 0, s, static_cast<bf16*>(values), count);
    else return cudaErrorInvalidValue;
    return tau_launch_status();
}

// values [rows, width] float, in place: exp(-exp(values + offset[column])).
TAU_EXPORT int tau_channel_decay(float* values, const float* offset, long long rows, int width, void* stream) {
    if (rows <= 0) return 0;
    if (!values || !offset || width <= 0) return cudaErrorInvalidValue;
    const long long count = rows * width;
    const unsigned blocks = static_cast<unsigned>((count + 255) / 256 < 1184 ? (count + 255) / 256 : 1184);
    tau_launch(channel_decay_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream), values, offset, count, width);
    return tau_launch_status();
}

// state: [heads, value_dim, key_dim] floats per slot, slots `slot_stride` apart.
TAU_EXPORT int tau_wkv(const float* r, const float* k, const float* v, const float* w, const float* bonus, float* state, long long slot_stride,
                       const int* cu_seqlens, const int* seq_slot, float* out, int n_seqs, int heads, int value_dim, void* stream) {
    if (n_seqs <= 0) return 0;
    if (!r || !k || !v || !w || !bonus || !state || !cu_seqlens || !seq_slot || !out || heads <= 0 || value_dim <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Value columns to a block: 32 where that many blocks fill the machine, else 16 (blocks of 8 and 4 columns were slower: every block
    // brings the head's r, k and w for itself, and that, not the walk, is then a block's work).
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const int tile = static_cast<long long>(heads) * n_seqs * ((value_dim + 31) / 32) < sms ? 16 : 32;
    dim3 grid(heads, n_seqs, (value_dim + tile - 1) / tile), block(tile * kSplit);
#define TAU_WKV(COLUMNS) tau_launch(wkv_kernel<COLUMNS>, grid, block, 0, s, r, k, v, w, bonus, state, slot_stride, cu_seqlens, seq_slot, out, heads, value_dim)
    if (tile == 32) TAU_WKV(32);
    else TAU_WKV(16);
#undef TAU_WKV
    return tau_launch_status();
}
