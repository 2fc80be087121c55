// The gated delta rule: a matrix state S (key_dim x value_dim) per head that decays, is corrected towards the token's value along
// the token's key, and is read with the token's query:
//
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q            (the read-out sees the token's own write)
//
// `q` and `k` belong to key heads (value head h reads key head h / (heads / key_heads)); q and k are unit vectors per head
// (x / sqrt(sum x^2 + 1e-6)), q also times key_dim^-1/2; beta = sigmoid(b); g = exp(-exp(A_log) softplus(a + dt_bias)).
//
//   prepare:  per token, in 32-bit and in place on [q | k | v] rows: the two unit norms and the query's scale, k . q per key head,
//             and (g, beta) per value head from the pre-activations.
//   walk:     one block owns (sequence, head, tile of value columns) and walks the run's tokens in order; what the next few tokens
//             bring (q, k, the tile's values, g, beta, k . q) is on its way into a ring in shared memory meanwhile (cp.async), so that
//             a token waits for shared memory and one barrier, not for a round trip to memory.  A column of S is shared by
//             kSplit threads, each with kRows key rows in registers.  With a = S_old^T k and b = S_old^T q (both from the state
//             before the token, one pass and one barrier) the token's result is u = beta (v - g a), o = g b + u (k . q),
//             S = g S_old + k u^T: the equations above with the decay pulled out of the sums.
//
// A decay per head and key channel (`channel`: g is a vector over the rows of S, from pre-activations [tokens, heads * key_dim]) walks the
// same way with the vector inside the sums: a = S_old^T (g * k), b = S_old^T (g * q), u = beta (v - a), o = b + u (k . q),
// S = g * S_old + k u^T.
//
// The state is 32-bit and lives in the cache, [heads, value_dim, key_dim] per slot.  TAU_KEY_DIM fixes key_dim.
#include "common.cuh"

#ifndef TAU_KEY_DIM
#error "compile with -DTAU_KEY_DIM=<key elements per head>"
#endif

namespace {

constexpr int kDim = TAU_KEY_DIM;
constexpr int kSplit = kDim <= 16 ? 1 : kDim <= 32 ? 2 : kDim <= 64 ? 4 : kDim <= 128 ? 8 : kDim <= 256 ? 16 : 32;   // threads that share a column
constexpr int kRows = (kDim + kSplit - 1) / kSplit;
constexpr bool kExact = kDim % kSplit == 0;      // every thread's rows exist

// grid: tokens; block: 128.  rows [tokens, stride] float: q at q_offset (key_heads * kDim), k at k_offset.  pre [tokens, pre_stride]:
// the pre-activations of beta, then (without `channel`) of the decay's step.  gates [tokens, heads, 2] = (g, beta); kq [tokens, key_heads].
// `channel` [tokens, heads * kDim]: the pre-activations of a decay per head and key channel (dt_bias is then as wide), replaced by the
// decays themselves; g of `gates` is then 1.
__global__ void __launch_bounds__(128)
delta_prepare_kernel(float* __restrict__ rows, long long stride, int q_offset, int k_offset, const float* __restrict__ pre, int pre_stride,
                     const float* __restrict__ a_log, const float* __restrict__ dt_bias, float* __restrict__ gates, float* __restrict__ kq,
                     float* __restrict__ channel, int heads, int key_heads, float query_scale) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int token = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    float* row = rows + static_cast<size_t>(token) * stride;
    for (int head = warp; head < key_heads; head += warps) {
        float* q = row + q_offset + head * kDim;
        float* k = row + k_offset + head * kDim;
        float qq = 0.0f, kk = 0.0f;
        for (int d = lane; d < kDim; d += 32) {
            qq = fmaf(q[d], q[d], qq);
            kk = fmaf(k[d], k[d], kk);
        }
        const float q_factor = query_scale / sqrtf(warp_sum(qq) + 1e-6f), k_factor = 1.0f / sqrtf(warp_sum(kk) + 1e-6f);
        float dot = 0.0f;
        for (int d = lane; d < kDim; d += 32) {
            const float a = q[d] * q_factor, b = k[d] * k_factor;
            q[d] = a;
            k[d] = b;
            dot = fmaf(a, b, dot);
        }
        dot = warp_sum(dot);
        if (lane == 0) kq[static_cast<size_t>(token) * key_heads + head] = dot;
    }
    for (int head = threadIdx.x; head < heads; head += blockDim.x) {
        const float b = pre[static_cast<size_t>(token) * pre_stride + head];
        float decay = 1.0f;
        if (!channel) {
            const float z = pre[static_cast<size_t>(token) * pre_stride + heads + head] + dt_bias[head];
            const float soft = z > 20.0f ? z : log1pf(expf(z));
            decay = expf(-expf(a_log[head]) * soft);
        }
        gates[(static_cast<size_t>(token) * heads + head) * 2] = decay;
        gates[(static_cast<size_t>(token) * heads + head) * 2 + 1] = 1.0f / (1.0f + expf(-b));
    }
    if (channel) {
        float* steps = channel + static_cast<size_t>(token) * heads * kDim;
        for (int index = threadIdx.x; index < heads * kDim; index += blockDim.x) {
            const float z = steps[index] + dt_bias[index];
            const float soft = z > 20.0f ? z : log1pf(expf(z));
            steps[index] = expf(-expf(a_log[index / kDim]) * soft);
        }
    }
}

// Four bytes from global to shared memory without passing a register; complete after `copy_wait` and a barrier.
__device__ __forceinline__ void copy_float(float* target, const float* source) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(target))), "l"(source) : "memory");
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int kRing = kDim <= 256 ? 8 : 4;      // tokens whose q, k, values and gates are in shared memory or on their way there

template <int kColumns, bool kChannel>
__global__ void __launch_bounds__(kColumns * kSplit)
delta_rule_kernel(const float* __restrict__ rows, long long stride, int q_offset, int k_offset, int v_offset, const float* __restrict__ gates,
                  const float* __restrict__ kq, const float* __restrict__ channel, float* __restrict__ state, long long slot_stride,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, float* __restrict__ out, int heads, int key_heads, int value_dim) {
    grid_dependents_launch();
    grid_dependency_wait();
    __shared__ __align__(16) float qs[kRing][kDim], ks[kRing][kDim];      // a thread's rows start on 16 bytes where kRows is a multiple of 4
    __shared__ __align__(16) float gs[kRing][kChannel ? kDim : 1];        // the head's decay per key channel
    __shared__ float vs[kRing][kColumns], scalars[kRing][4], part_a[2][kSplit][kColumns], part_b[2][kSplit][kColumns];
    const int head = blockIdx.x, sequence = blockIdx.y, key_head = head / (heads / key_heads);
    const int local = threadIdx.x % kColumns, part = threadIdx.x / kColumns, row0 = part * kRows;
    const int column = blockIdx.z * kColumns + local;
    const bool live = column < value_dim;
    float* record = state + static_cast<size_t>(seq_slot[sequence]) * slot_stride + (static_cast<size_t>(head) * value_dim + (live ? column : 0)) * kDim;
    float S[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) S[r] = (live && row0 + r < kDim) ? record[row0 + r] : 0.0f;
    const int begin = cu_seqlens[sequence], end = cu_seqlens[sequence + 1];
    constexpr int kStage = (kDim + kColumns * kSplit - 1) / (kColumns * kSplit);
    // Asks for token `begin + index` (if the run has it) in its place of the ring; one group of copies per token, empty ones too, so
    // that the count of groups in flight says which tokens have arrived.
    auto stage = [&](int index) {
        const int token = begin + index, place = index % kRing;
        if (token < end) {
            const float* row = rows + static_cast<size_t>(token) * stride;
#pragma unroll
            for (int i = 0; i < kStage; ++i) {
                const int d = threadIdx.x + i * kColumns * kSplit;
                if (d < kDim) {
                    copy_float(&qs[place][d], row + q_offset + key_head * kDim + d);
                    copy_float(&ks[place][d], row + k_offset + key_head * kDim + d);
                    if (kChannel) copy_float(&gs[place][d], channel + (static_cast<size_t>(token) * heads + head) * kDim + d);
                }
            }
            if (part == 0 && live) copy_float(&vs[place][local], row + v_offset + head * value_dim + column);
            if (threadIdx.x < 2) copy_float(&scalars[place][threadIdx.x], gates + (static_cast<size_t>(token) * heads + head) * 2 + threadIdx.x);
            if (threadIdx.x == 2) copy_float(&scalars[place][2], kq + static_cast<size_t>(token) * key_heads + key_head);
        }
        copy_commit();
    };
#pragma unroll
    for (int index = 0; index < kRing - 1; ++index) stage(index);
    copy_wait<kRing - 2>();      // the first token has arrived
    __syncthreads();
    for (int token = begin; token < end; ++token) {
        const int index = token - begin, place = index % kRing, half = index & 1;
        const float value = live ? vs[place][local] : 0.0f;
        const float decay = scalars[place][0], beta = scalars[place][1], key_query = scalars[place][2];
        float key[kRows], keep[kChannel ? kRows : 1];
        float a[2] = {0.0f, 0.0f}, b[2] = {0.0f, 0.0f};
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            key[r] = (kExact || row0 + r < kDim) ? ks[place][row0 + r] : 0.0f;
            const float query = (kExact || row0 + r < kDim) ? qs[place][row0 + r] : 0.0f;
            if (kChannel) {
                keep[r] = (kExact || row0 + r < kDim) ? gs[place][row0 + r] : 0.0f;
                const float kept = keep[r] * S[r];
                a[r & 1] = fmaf(kept, key[r], a[r & 1]);
                b[r & 1] = fmaf(kept, query, b[r & 1]);
            } else {
                a[r & 1] = fmaf(S[r], key[r], a[r & 1]);
                b[r & 1] = fmaf(S[r], query, b[r & 1]);
            }
        }
        part_a[half][part][local] = a[0] + a[1];
        part_b[half][part][local] = b[0] + b[1];
        // The place of the token before this one is free: everybody has passed that token's barrier, and read its place before it.
        stage(index + kRing - 1);
        copy_wait<kRing - 2>();      // this thread's copies of the next token are done; the barrier shows everybody's
        __syncthreads();
        float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
        for (int p = 0; p < kSplit; ++p) {
            sum_a += part_a[half][p][local];
            sum_b += part_b[half][p][local];
        }
        const float update = beta * (value - decay * sum_a);
#pragma unroll
        for (int r = 0; r < kRows; ++r) S[r] = fmaf(kChannel ? keep[r] : decay, S[r], key[r] * update);
        if (part == 0 && live) out[(static_cast<size_t>(token) * heads + head) * value_dim + column] = fmaf(decay, sum_b, update * key_query);
    }
    copy_wait<0>();
    if (live) {
#pragma unroll
        for (int r = 0; r < kRows; ++r)
            if (row0 + r < kDim) record[row0 + r] = S[r];
    }
}

}  // namespace

TAU_EXPORT int tau_delta_key_dim() { return kDim; }

TAU_EXPORT int tau_delta_prepare(float* rows, long long stride, int q_offset, int k_offset, const float* pre, int pre_stride, const float* a_log,
                                 const float* dt_bias, float* gates, float* kq, float* channel, int tokens, int heads, int key_heads, float query_scale,
                                 void* stream) {
    if (tokens <= 0) return 0;
    if (!rows || !pre || !a_log || !dt_bias || !gates || !kq || heads <= 0 || key_heads <= 0 || heads % key_heads != 0 || pre_stride < (channel ? heads : 2 * heads))
        return cudaErrorInvalidValue;
    tau_launch(delta_prepare_kernel, dim3(tokens), dim3(128), 0, static_cast<cudaStream_t>(stream), rows, stride, q_offset, k_offset, pre, pre_stride, a_log,
               dt_bias, gates, kq, channel, heads, key_heads, query_scale);
    return tau_launch_status();
}

// rows [tokens, stride] float with q, k (key_heads * key_dim each) and v (heads * value_dim) at their offsets, prepared as above.
// state: [heads, value_dim, key_dim] floats per slot, slots `slot_stride` apart.  out [tokens, heads * value_dim].
// `channel` (or null): [tokens, heads * key_dim], a decay per head and key channel as `tau_delta_prepare` left it.
TAU_EXPORT int tau_delta_rule(const float* rows, long long stride, int q_offset, int k_offset, int v_offset, const float* gates, const float* kq,
                              const float* channel, float* state, long long slot_stride, const int* cu_seqlens, const int* seq_slot, float* out, int n_seqs, int heads,
                              int key_heads, int value_dim, void* stream) {
    if (n_seqs <= 0) return 0;
    if (!rows || !gates || !kq || !state || !cu_seqlens || !seq_slot || !out || heads <= 0 || key_heads <= 0 || heads % key_heads != 0 || value_dim <= 0)
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool narrow = heads * n_seqs * ((value_dim + 31) / 32) < 148 && kSplit <= 16;     // blocks of 16 columns reach more SMs
    const int tile = narrow ? 16 : 32;
    dim3 grid(heads, n_seqs, (value_dim + tile - 1) / tile), block(tile * kSplit);
#define TAU_DELTA(COLUMNS, CHANNEL)                                                                                                               \
    tau_launch(delta_rule_kernel<COLUMNS, CHANNEL>, grid, block, 0, s, rows, stride, q_offset, k_offset, v_offset, gates, kq, channel, state, slot_stride, \
               cu_seqlens, seq_slot, out, heads, key_heads, value_dim)
    if (narrow) {
        if (channel) TAU_DELTA(16, true); else TAU_DELTA(16, false);
    } else {
        if (channel) TAU_DELTA(32, true); else TAU_DELTA(32, false);
    }
#undef TAU_DELTA
    return tau_launch_status();
}
