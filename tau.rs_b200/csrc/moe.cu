// Routed experts, token by token: a router that scores the experts in 32-bit and picks `top` of them, the chosen
// experts' gated products, and the weighted sum of their outputs (plus a shared expert's, scaled by its own gate).
//
//   route:    z = W_router h + bias (32-bit weights and sums; the bias is optional); s = sigmoid(z) or softmax(z); the `top` largest of
//             s + correction are chosen (the lowest index among equals), their weights are s itself, divided by
//             their sum if `renormalize`; shared_gate = sigmoid(w_sg . h).
//   gate_up:  inner[token, place] = silu(W_gate[e] h) * (W_up[e] h) for the expert e of each (token, place).
//   down:     out[token] = sum over places of weight * (W_down[e] inner[token, place]) + shared_gate * shared[token], 32-bit.
//
// Experts numbered `real_experts` and up have no weights: they return what they read (identity experts), so a pair that chose one adds
// weight * h to the token's sum.
//
// These are weight-streaming kernels: a warp per output feature, the activation row in shared memory as floats.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

// Dot product of a weight row with a float vector in shared memory, over the warp.
template <typename T>
__device__ __forceinline__ float warp_dot(const T* __restrict__ weights, const float* __restrict__ vector, int length, int lane) {
    float sum = 0.0f;
    for (int column = lane; column < length; column += 32) sum = fmaf(to_float(weights[column]), vector[column], sum);
    return warp_sum(sum);
}

// 32-bit rows (the router's) that start on a 16-byte boundary are read four elements at a time.
template <>
__device__ __forceinline__ float warp_dot<float>(const float* __restrict__ weights, const float* __restrict__ vector, int length, int lane) {
    float sum = 0.0f;
    if ((reinterpret_cast<uintptr_t>(weights) & 15) == 0 && length % 4 == 0) {
        float other = 0.0f;
        int column = lane * 4;
        for (; column + 128 < length; column += 256) {
            const float4 w0 = *reinterpret_cast<const float4*>(weights + column), w1 = *reinterpret_cast<const float4*>(weights + column + 128);
            const float4 x0 = *reinterpret_cast<const float4*>(vector + column), x1 = *reinterpret_cast<const float4*>(vector + column + 128);
            sum = fmaf(w0.x, x0.x, fmaf(w0.y, x0.y, fmaf(w0.z, x0.z, fmaf(w0.w, x0.w, sum))));
            other = fmaf(w1.x, x1.x, fmaf(w1.y, x1.y, fmaf(w1.z, x1.z, fmaf(w1.w, x1.w, other))));
        }
        if (column < length) {
            const float4 w0 = *reinterpret_cast<const float4*>(weights + column), x0 = *reinterpret_cast<const float4*>(vector + column);
            sum = fmaf(w0.x, x0.x, fmaf(w0.y, x0.y, fmaf(w0.z, x0.z, fmaf(w0.w, x0.w, sum))));
        }
        sum += other;
    } else {
        for (int column = lane; column < length; column += 32) sum = fmaf(weights[column], vector[column], sum);
    }
    return warp_sum(sum);
}

// Eight bfloat16 weights against eight floats of shared memory, which are read as two 16-byte words (lanes 32 bytes apart meet
// two to a bank that way, not eight).
__device__ __forceinline__ float dot8(const uint4& raw, const float* __restrict__ vector) {
    const float4 low = *reinterpret_cast<const float4*>(vector), high = *reinterpret_cast<const float4*>(vector + 4);
    float sum = __uint_as_float(raw.x << 16) * low.x;
    sum = fmaf(__uint_as_float(raw.x & 0xffff0000u), low.y, sum);
    sum = fmaf(__uint_as_float(raw.y << 16), low.z, sum);
    sum = fmaf(__uint_as_float(raw.y & 0xffff0000u), low.w, sum);
    sum = fmaf(__uint_as_float(raw.z << 16), high.x, sum);
    sum = fmaf(__uint_as_float(raw.z & 0xffff0000u), high.y, sum);
    sum = fmaf(__uint_as_float(raw.w << 16), high.z, sum);
    sum = fmaf(__uint_as_float(raw.w & 0xffff0000u), high.w, sum);
    return sum;
}

// bfloat16 rows that start on a 16-byte boundary are read eight elements at a time.
template <>
__device__ __forceinline__ float warp_dot<bf16>(const bf16* __restrict__ weights, const float* __restrict__ vector, int length, int lane) {
    float sum = 0.0f;
    if ((reinterpret_cast<uintptr_t>(weights) & 15) == 0 && length % 8 == 0) {
        for (int column = lane * 8; column < length; column += 256) sum += dot8(*reinterpret_cast<const uint4*>(weights + column), vector + column);
    } else {
        for (int column = lane; column < length; column += 32) sum = fmaf(__bfloat162float(weights[column]), vector[column], sum);
    }
    return warp_sum(sum);
}

// Two dot products at once (a gate row and its up row, or the rows of two places), so that a lane has four 16-byte loads in
// flight where the rows allow them.
template <typename T>
__device__ __forceinline__ void warp_dot_pair(const T* __restrict__ first, const float* __restrict__ first_vector, const T* __restrict__ second,
                                              const float* __restrict__ second_vector, int length, int lane, float& first_sum, float& second_sum) {
    first_sum = warp_dot(first, first_vector, length, lane);
    second_sum = warp_dot(second, second_vector, length, lane);
}

template <>
__device__ __forceinline__ void warp_dot_pair<bf16>(const bf16* __restrict__ first, const float* __restrict__ first_vector, const bf16* __restrict__ second,
                                                    const float* __restrict__ second_vector, int length, int lane, float& first_sum, float& second_sum) {
    if (((reinterpret_cast<uintptr_t>(first) | reinterpret_cast<uintptr_t>(second)) & 15) != 0 || length % 8 != 0) {
        first_sum = warp_dot(first, first_vector, length, lane);
        second_sum = warp_dot(second, second_vector, length, lane);
        return;
    }
    float a = 0.0f, b = 0.0f, c = 0.0f, d = 0.0f;
    int column = lane * 8;
    for (; column + 768 < length; column += 1024) {      // eight loads in flight
        uint4 x[4], y[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[i] = *reinterpret_cast<const uint4*>(first + column + 256 * i);
            y[i] = *reinterpret_cast<const uint4*>(second + column + 256 * i);
        }
        a += dot8(x[0], first_vector + column) + dot8(x[2], first_vector + column + 512);
        b += dot8(y[0], second_vector + column) + dot8(y[2], second_vector + column + 512);
        c += dot8(x[1], first_vector + column + 256) + dot8(x[3], first_vector + column + 768);
        d += dot8(y[1], second_vector + column + 256) + dot8(y[3], second_vector + column + 768);
    }
    for (; column + 256 < length; column += 512) {
        const uint4 a0 = *reinterpret_cast<const uint4*>(first + column), b0 = *reinterpret_cast<const uint4*>(second + column);
        const uint4 a1 = *reinterpret_cast<const uint4*>(first + column + 256), b1 = *reinterpret_cast<const uint4*>(second + column + 256);
        a += dot8(a0, first_vector + column);
        b += dot8(b0, second_vector + column);
        c += dot8(a1, first_vector + column + 256);
        d += dot8(b1, second_vector + column + 256);
    }
    if (column < length) {
        const uint4 a0 = *reinterpret_cast<const uint4*>(first + column), b0 = *reinterpret_cast<const uint4*>(second + column);
        a += dot8(a0, first_vector + column);
        b += dot8(b0, second_vector + column);
    }
    first_sum = warp_sum(a + c);
    second_sum = warp_sum(b + d);
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
moe_route_kernel(const T* __restrict__ hidden, const float* __restrict__ router, const float* __restrict__ logit_bias, const float* __restrict__ correction,
                 const float* __restrict__ shared_gate_weight, int* __restrict__ chosen, float* __restrict__ weights, float* __restrict__ shared_gate,
                 int width, int experts, int top, int softmax, int renormalize) {
    grid_dependents_launch();
    grid_dependency_wait();
    extern __shared__ __align__(16) float shared[];
    float* row = shared;               // [width]
    float* scores = shared + width;    // [experts]
    float* choice = scores + experts;  // [experts]
    const int token = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int column = threadIdx.x; column < width; column += blockDim.x) row[column] = to_float(hidden[static_cast<size_t>(token) * width + column]);
    __syncthreads();
    for (int expert = warp; expert < experts; expert += kWarps) {
        const float z = warp_dot(router + static_cast<size_t>(expert) * width, row, width, lane);
        if (lane == 0) scores[expert] = z + (logit_bias ? logit_bias[expert] : 0.0f);
    }
    if (shared_gate_weight && warp == kWarps - 1) {
        const float z = warp_dot(shared_gate_weight, row, width, lane);
        if (lane == 0) shared_gate[token] = 1.0f / (1.0f + expf(-z));
    }
    __syncthreads();
    if (warp != 0) return;
    if (softmax) {
        float top_z = -INFINITY;
        for (int expert = lane; expert < experts; expert += 32) top_z = fmaxf(top_z, scores[expert]);
        top_z = warp_max(top_z);
        float total = 0.0f;
        for (int expert = lane; expert < experts; expert += 32) total += expf(scores[expert] - top_z);
        total = warp_sum(total);
        for (int expert = lane; expert < experts; expert += 32) scores[expert] = expf(scores[expert] - top_z) / total;
    } else {
        for (int expert = lane; expert < experts; expert += 32) scores[expert] = 1.0f / (1.0f + expf(-scores[expert]));
    }
    for (int expert = lane; expert < experts; expert += 32) choice[expert] = scores[expert] + (correction ? correction[expert] : 0.0f);
    __syncwarp();
    float total = 0.0f;
    for (int place = 0; place < top; ++place) {
        float best = -INFINITY;
        int best_expert = 0x7fffffff;
        for (int expert = lane; expert < experts; expert += 32) {
            const float value = choice[expert];
            if (value > best) { best = value; best_expert = expert; }   // ascending scan: the lowest index among equals stays
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, best, offset);
            const int other_expert = __shfl_xor_sync(0xffffffffu, best_expert, offset);
            if (other > best || (other == best && other_expert < best_expert)) { best = other; best_expert = other_expert; }
        }
        if (best_expert >= experts) best_expert = place;     // only rows of NaN come here
        if (lane == 0) {
            chosen[static_cast<size_t>(token) * top + place] = best_expert;
            weights[static_cast<size_t>(token) * top + place] = scores[best_expert];
            choice[best_expert] = -INFINITY;
        }
        total += scores[best_expert];
        __syncwarp();
    }
    if (renormalize && lane == 0)
        for (int place = 0; place < top; ++place) weights[static_cast<size_t>(token) * top + place] /= total;
}

// grid (token-place pairs, feature tiles).  gate_up: [experts, 2 * inner, width], gate rows first.
template <typename T>
__global__ void __launch_bounds__(kThreads)
moe_gate_up_kernel(const T* __restrict__ hidden, const T* __restrict__ gate_up, const int* __restrict__ chosen, const float* __restrict__ input_weights,
                   T* __restrict__ inner_out, int width, int inner, int top, int features_per_block, int interleave, int real_experts) {
    grid_dependents_launch();
    grid_dependency_wait();
    extern __shared__ __align__(16) float row[];
    const int pair = blockIdx.x, token = pair / top, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (chosen[pair] >= real_experts) return;      // an identity expert has no inner features
    for (int column = threadIdx.x; column < width; column += blockDim.x) row[column] = to_float(hidden[static_cast<size_t>(token) * width + column]);
    __syncthreads();
    const T* weights = gate_up + static_cast<size_t>(chosen[pair]) * 2 * inner * width;
    // A weight on the expert's input: both products are linear in the row, so the weight multiplies their 32-bit sums.
    const float input_weight = input_weights ? input_weights[pair] : 1.0f;
    const int begin = blockIdx.y * features_per_block, end = min(inner, begin + features_per_block);
    for (int feature = begin + warp; feature < end; feature += kWarps) {
        // Plain: gate rows, then up rows.  Interleaved: groups of `interleave` gate rows, each followed by its up rows.
        const int gate_row = interleave ? feature / interleave * 2 * interleave + feature % interleave : feature;
        const int up_row = interleave ? gate_row + interleave : inner + feature;
        float gate, up;
        warp_dot_pair(weights + static_cast<size_t>(gate_row) * width, row, weights + static_cast<size_t>(up_row) * width, row, width, lane, gate, up);
        gate *= input_weight;
        up *= input_weight;
        if (lane == 0) inner_out[static_cast<size_t>(pair) * inner + feature] = from_float<T>(gate / (1.0f + expf(-gate)) * up);
    }
}

// grid (tokens, feature tiles).  down: [experts, width, inner].
template <typename T>
__global__ void __launch_bounds__(kThreads)
moe_down_kernel(const T* __restrict__ inner_in, const T* __restrict__ down, const int* __restrict__ chosen, const float* __restrict__ weights,
                const T* __restrict__ shared_out, const float* __restrict__ shared_gate, float* __restrict__ out, int width, int inner, int top,
                int features_per_block, const T* __restrict__ hidden, int real_experts) {
    grid_dependents_launch();
    grid_dependency_wait();
    extern __shared__ __align__(16) float rows[];     // [top][inner]
    const int token = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int item = threadIdx.x; item < top * inner; item += blockDim.x)      // an identity expert's place was never written: nothing of it is read
        rows[item] = chosen[static_cast<size_t>(token) * top + item / inner] < real_experts ? to_float(inner_in[static_cast<size_t>(token) * top * inner + item]) : 0.0f;
    __syncthreads();
    const int begin = blockIdx.y * features_per_block, end = min(width, begin + features_per_block);
    for (int feature = begin + warp; feature < end; feature += kWarps) {
        float sum = 0.0f;
        int place = 0;
        // What one place adds: its expert's row against the place's inner features, or the token's own feature for an identity expert.
        auto alone = [&](int at) {
            const int expert = chosen[static_cast<size_t>(token) * top + at];
            if (expert >= real_experts) return hidden ? to_float(hidden[static_cast<size_t>(token) * width + feature]) : 0.0f;
            return warp_dot(down + (static_cast<size_t>(expert) * width + feature) * inner, rows + at * inner, inner, lane);
        };
        for (; place + 1 < top; place += 2) {     // two places at a time, summed in place order
            const int e0 = chosen[static_cast<size_t>(token) * top + place], e1 = chosen[static_cast<size_t>(token) * top + place + 1];
            float a, b;
            if (e0 < real_experts && e1 < real_experts) {
                const T* first = down + (static_cast<size_t>(e0) * width + feature) * inner;
                const T* second = down + (static_cast<size_t>(e1) * width + feature) * inner;
                warp_dot_pair(first, rows + place * inner, second, rows + (place + 1) * inner, inner, lane, a, b);
            } else {
                a = alone(place);
                b = alone(place + 1);
            }
            sum = fmaf(weights ? weights[static_cast<size_t>(token) * top + place] : 1.0f, a, sum);
            sum = fmaf(weights ? weights[static_cast<size_t>(token) * top + place + 1] : 1.0f, b, sum);
        }
        if (place < top) sum = fmaf(weights ? weights[static_cast<size_t>(token) * top + place] : 1.0f, alone(place), sum);
        if (lane == 0) {
            if (shared_out) sum += (shared_gate ? shared_gate[token] : 1.0f) * to_float(shared_out[static_cast<size_t>(token) * width + feature]);
            out[static_cast<size_t>(token) * width + feature] = sum;
        }
    }
}

// The (token, place) pairs grouped by expert, by one block: offsets[e] .. offsets[e + 1] are the places of expert e's pairs in
// `order`; position[pair] is where a pair went.  The order inside a group depends on timing; nothing computed from it does.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ chosen, int pairs, int experts, int* __restrict__ offsets, int* __restrict__ order, int* __restrict__ position) {
    grid_dependents_launch();
    grid_dependency_wait();
    extern __shared__ int counters[];       // [experts] counts, then [experts] cursors
    int* cursor = counters + experts;
    for (int expert = threadIdx.x; expert < experts; expert += blockDim.x) counters[expert] = 0;
    __syncthreads();
    for (int pair = threadIdx.x; pair < pairs; pair += blockDim.x) atomicAdd(&counters[chosen[pair]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int total = 0;
        for (int expert = 0; expert < experts; ++expert) {
            offsets[expert] = total;
            cursor[expert] = total;
            total += counters[expert];
        }
        offsets[experts] = total;
    }
    __syncthreads();
    for (int pair = threadIdx.x; pair < pairs; pair += blockDim.x) {
        const int place = atomicAdd(&cursor[chosen[pair]], 1);
        order[place] = pair;
        position[pair] = place;
    }
}

// gathered[i] = hidden[order[i] / top] (times input_weights[order[i]], if given): the rows of each expert's tokens side by side.
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ hidden, const int* __restrict__ order, const float* __restrict__ input_weights, T* __restrict__ gathered,
                                  int width, int top) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int pair = order[blockIdx.x];
    const T* source = hidden + static_cast<size_t>(pair / top) * width;
    T* target = gathered + static_cast<size_t>(blockIdx.x) * width;
    if (input_weights) {
        const float weight = input_weights[pair];
        for (int column = threadIdx.x; column < width; column += blockDim.x) target[column] = from_float<T>(weight * to_float(source[column]));
    } else {
        for (int column = threadIdx.x; column < width; column += blockDim.x) target[column] = source[column];
    }
}

// out[token] = sum over places of weight * rows[position[token, place]] + shared_gate * shared[token], in place order.
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ rows, const int* __restrict__ position, const float* __restrict__ weights,
                                   const T* __restrict__ shared_out, const float* __restrict__ shared_gate, float* __restrict__ out, int width, int top,
                                   const int* __restrict__ chosen, const T* __restrict__ hidden, int real_experts) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int token = blockIdx.x;
    for (int column = threadIdx.x; column < width; column += blockDim.x) {
        float sum = 0.0f;
        for (int place = 0; place < top; ++place) {
            const size_t pair = static_cast<size_t>(token) * top + place;
            const bool identity = chosen && chosen[pair] >= real_experts;      // such a pair's row was never computed
            const float row = identity ? to_float(hidden[static_cast<size_t>(token) * width + column]) : rows[static_cast<size_t>(position[pair]) * width + column];
            sum = fmaf(weights ? weights[pair] : 1.0f, row, sum);
        }
        if (shared_out) sum += (shared_gate ? shared_gate[token] : 1.0f) * to_float(shared_out[static_cast<size_t>(token) * width + column]);
        out[static_cast<size_t>(token) * width + column] = sum;
    }
}

template <typename T>
int launch_all(int what, const void* a, const void* b, const void* c, const void* d, const void* e, const void* f, void* o1, void* o2, void* o3,
               int tokens, int width, int inner, int experts, int top, int flag_a, int flag_b, cudaStream_t s, const void* g = nullptr) {
    if (what == 0) {
        const size_t bytes = (static_cast<size_t>(width) + 2 * experts) * sizeof(float);
        if (bytes > 48 * 1024 && cudaFuncSetAttribute(moe_route_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) != cudaSuccess)
            return cudaErrorInvalidValue;
        tau_launch(moe_route_kernel<T>, dim3(tokens), dim3(kThreads), bytes, s, static_cast<const T*>(a), static_cast<const float*>(b), static_cast<const float*>(e),
                   static_cast<const float*>(c), static_cast<const float*>(d), static_cast<int*>(o1), static_cast<float*>(o2), static_cast<float*>(o3), width, experts, top, flag_a, flag_b);
    } else if (what == 1) {
        const int per_block = 64;
        const size_t bytes = static_cast<size_t>(width) * sizeof(float);
        if (bytes > 48 * 1024 && cudaFuncSetAttribute(moe_gate_up_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) != cudaSuccess)
            return cudaErrorInvalidValue;
        tau_launch(moe_gate_up_kernel<T>, dim3(tokens * top, (inner + per_block - 1) / per_block), dim3(kThreads), bytes, s, static_cast<const T*>(a),
                   static_cast<const T*>(b), static_cast<const int*>(c), static_cast<const float*>(d), static_cast<T*>(o1), width, inner, top, per_block, flag_a, experts);
    } else {
        const int per_block = tokens * ((width + 63) / 64) >= 1024 ? 64 : tokens * ((width + 31) / 32) >= 1024 ? 32 : 16;   // few tokens: smaller tiles, more blocks
        const size_t bytes = static_cast<size_t>(top) * inner * sizeof(float);
        if (bytes > 48 * 1024 && cudaFuncSetAttribute(moe_down_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) != cudaSuccess)
            return cudaErrorInvalidValue;
        tau_launch(moe_down_kernel<T>, dim3(tokens, (width + per_block - 1) / per_block), dim3(kThreads), bytes, s, static_cast<const T*>(a), static_cast<const T*>(b),
                   static_cast<const int*>(c), static_cast<const float*>(d), static_cast<const T*>(e), static_cast<const float*>(f), static_cast<float*>(o1),
                   width, inner, top, per_block, static_cast<const T*>(g), experts);
    }
    return tau_launch_status();
}

}  // namespace

TAU_EXPORT int tau_moe_route(int dtype, const void* hidden, const float* router, const float* logit_bias, const float* correction, const float* shared_gate_weight, int* chosen,
                             float* weights, float* shared_gate, int tokens, int width, int experts, int top, int softmax, int renormalize, void* stream) {
    if (tokens <= 0) return 0;
    if (!hidden || !router || !chosen || !weights || width <= 0 || experts <= 0 || top <= 0 || top > experts || (shared_gate_weight && !shared_gate))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TAU_F32) return launch_all<float>(0, hidden, router, correction, shared_gate_weight, logit_bias, nullptr, chosen, weights, shared_gate, tokens, width, 0, experts, top, softmax, renormalize, s);
    if (dtype == TAU_BF16) return launch_all<bf16>(0, hidden, router, correction, shared_gate_weight, logit_bias, nullptr, chosen, weights, shared_gate, tokens, width, 0, experts, top, softmax, renormalize, s);
    return cudaErrorInvalidValue;
}

// `real_experts`: experts with weights (gate_up holds that many); a pair that chose a higher number is left alone.
TAU_EXPORT int tau_moe_gate_up(int dtype, const void* hidden, const void* gate_up, const int* chosen, const float* input_weights, void* inner_out, int tokens,
                               int width, int inner, int top, int interleave, int real_experts, void* stream) {
    if (tokens <= 0) return 0;
    if (!hidden || !gate_up || !chosen || !inner_out || width <= 0 || inner <= 0 || top <= 0 || static_cast<long long>(tokens) * top > 0x7fffffff) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TAU_F32) return launch_all<float>(1, hidden, gate_up, chosen, input_weights, nullptr, nullptr, inner_out, nullptr, nullptr, tokens, width, inner, real_experts, top, interleave, 0, s);
    if (dtype == TAU_BF16) return launch_all<bf16>(1, hidden, gate_up, chosen, input_weights, nullptr, nullptr, inner_out, nullptr, nullptr, tokens, width, inner, real_experts, top, interleave, 0, s);
    return cudaErrorInvalidValue;
}

TAU_EXPORT int tau_moe_down(int dtype, const void* inner_in, const void* down, const int* chosen, const float* weights, const void* shared_out,
                            const float* shared_gate, float* out, int tokens, int width, int inner, int top, const void* hidden, int real_experts,
                            void* stream) {
    if (tokens <= 0) return 0;
    if (!inner_in || !down || !chosen || !out || width <= 0 || inner <= 0 || top <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TAU_F32) return launch_all<float>(2, inner_in, down, chosen, weights, shared_out, shared_gate, out, nullptr, nullptr, tokens, width, inner, real_experts, top, 0, 0, s, hidden);
    if (dtype == TAU_BF16) return launch_all<bf16>(2, inner_in, down, chosen, weights, shared_out, shared_gate, out, nullptr, nullptr, tokens, width, inner, real_experts, top, 0, 0, s, hidden);
    return cudaErrorInvalidValue;
}

TAU_EXPORT int tau_moe_sort(const int* chosen, int pairs, int experts, int* offsets, int* order, int* position, void* stream) {
    if (pairs <= 0) return 0;
    if (!chosen || !offsets || !order || !position || experts <= 0 || experts > 4096) return cudaErrorInvalidValue;
    tau_launch(moe_sort_kernel, dim3(1), dim3(1024), static_cast<size_t>(2 * experts) * sizeof(int), static_cast<cudaStream_t>(stream), chosen, pairs, experts,
               offsets, order, position);
    return tau_launch_status();
}

TAU_EXPORT int tau_moe_gather(int dtype, const void* hidden, const int* order, const float* input_weights, void* gathered, int pairs, int width, int top,
                              void* stream) {
    if (pairs <= 0) return 0;
    if (!hidden || !order || !gathered || width <= 0 || top <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TAU_F32) tau_launch(moe_gather_kernel<float>, dim3(pairs), dim3(kThreads), 0, s, static_cast<const float*>(hidden), order, input_weights, static_cast<float*>(gathered), width, top);
    else if (dtype == TAU_BF16) tau_launch(moe_gather_kernel<bf16>, dim3(pairs), dim3(kThreads), 0, s, static_cast<const bf16*>(hidden), order, input_weights, static_cast<bf16*>(gathered), width, top);
    else return cudaErrorInvalidValue;
    return tau_launch_status();
}

TAU_EXPORT int tau_moe_combine(int dtype, const float* rows, const int* position, const float* weights, const void* shared_out, const float* shared_gate,
                               float* out, int tokens, int width, int top, const int* chosen, const void* hidden, int real_experts, void* stream) {
    if (tokens <= 0) return 0;
    if (!rows || !position || !out || width <= 0 || top <= 0 || (chosen && !hidden)) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TAU_F32) tau_launch(moe_combine_kernel<float>, dim3(tokens), dim3(kThreads), 0, s, rows, position, weights, static_cast<const float*>(shared_out), shared_gate, out, width, top, chosen, static_cast<const float*>(hidden), real_experts);
    else if (dtype == TAU_BF16) tau_launch(moe_combine_kernel<bf16>, dim3(tokens), dim3(kThreads), 0, s, rows, position, weights, static_cast<const bf16*>(shared_out), shared_gate, out, width, top, chosen, static_cast<const bf16*>(hidden), real_experts);
    else return cudaErrorInvalidValue;
    return tau_launch_status();
}
