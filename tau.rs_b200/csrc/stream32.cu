// A residual stream kept in 32-bit beside activations of another dtype: embedding rows widened to float, and the
// fused sum of up to two branches into the stream followed by RMSNorm, with the output in the activations' dtype.
// Also the gated output stage of mixers whose result is 32-bit: optional RMS norm per group, weight, sigmoid gate.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float load_as_float(const void* base, int code, size_t index) {
    return code == TAU_BF16 ? __bfloat162float(static_cast<const bf16*>(base)[index]) : static_cast<const float*>(base)[index];
}

template <typename T>
__global__ void embedding_f32_kernel(const int* __restrict__ tokens, const T* __restrict__ table, float* __restrict__ out, int width, int vocab, float scale) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int row = blockIdx.x;
    const int token = tokens[row];
    float* target = out + static_cast<size_t>(row) * width;
    const bool inside = token >= 0 && token < vocab;   // refused on the host already; never read outside the table
    const T* source = table + static_cast<size_t>(inside ? token : 0) * width;
    for (int column = threadIdx.x; column < width; column += blockDim.x) target[column] = inside ? to_float(source[column]) * scale : 0.0f;
}

// r = rows ? rows[i] : i.  sum = stream[r] + branch_scale * (a[r] + b[r]) in 32-bit; if `update` the sum replaces stream[r];
// out[i] = sum / sqrt(mean(sum^2) + eps) * weight, rounded once to T.  With `groups` > 1 the row is cut into that many equal
// consecutive pieces and each is divided by its own root mean square (a warp sums a piece's squares).
constexpr int kMaxNormGroups = 1024;

template <typename T>
__global__ void __launch_bounds__(kThreads)
stream_add_norm_kernel(float* __restrict__ stream, const void* __restrict__ a, int a_code, const void* __restrict__ b, int b_code,
                       const int* __restrict__ rows, const float* __restrict__ weight, T* __restrict__ out, int width, float eps, int update,
                       int groups, float branch_scale) {
    grid_dependents_launch();
    grid_dependency_wait();
    __shared__ float scratch[33];
    __shared__ float inverses[kMaxNormGroups];
    const int row = rows ? rows[blockIdx.x] : blockIdx.x;
    const size_t base = static_cast<size_t>(row) * width;
    auto joined = [&](int column) {
        float value = stream[base + column];
        if (a) {
            float branch = load_as_float(a, a_code, base + column);
            if (b) branch += load_as_float(b, b_code, base + column);
            value = fmaf(branch_scale, branch, value);
        }
        return value;
    };
    T* target = out + static_cast<size_t>(blockIdx.x) * width;
    if (groups > 1) {
        if (update && a) {
            for (int column = threadIdx.x; column < width; column += blockDim.x) stream[base + column] = joined(column);
            __syncthreads();      // the pieces below are summed by other threads than those that wrote them
        }
        const bool stored = update || !a;
        const int piece = width / groups, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
        for (int group = warp; group < groups; group += warps) {
            float squares = 0.0f;
            for (int column = group * piece + lane; column < (group + 1) * piece; column += 32) {
                const float value = stored ? stream[base + column] : joined(column);
                squares = fmaf(value, value, squares);
            }
            squares = warp_sum(squares);
            if (lane == 0) inverses[group] = 1.0f / sqrtf(squares / static_cast<float>(piece) + eps);
        }
        __syncthreads();
        for (int column = threadIdx.x; column < width; column += blockDim.x)
            target[column] = from_float<T>((stored ? stream[base + column] : joined(column)) * inverses[column / piece] * weight[column]);
        return;
    }
    float squares = 0.0f;
    for (int column = threadIdx.x; column < width; column += blockDim.x) {
        const float value = joined(column);
        if (update) stream[base + column] = value;
        squares += value * value;
    }
    const float inverse = 1.0f / sqrtf(block_sum(squares, scratch) / static_cast<float>(width) + eps);
    for (int column = threadIdx.x; column < width; column += blockDim.x) {
        const float value = (a && !update) ? joined(column) : stream[base + column];     // each thread reads back what it wrote itself
        target[column] = from_float<T>(value * inverse * weight[column]);
    }
}

// out[row] = left_scale * left[row] / rms(left[row]) * left_weight + right_scale * right[row] / rms(right[row]) * right_weight: two results
// that are normalised over their whole width, each with its own weight, before they are added (eps inside the roots); all 32-bit.
__global__ void __launch_bounds__(kThreads)
normed_pair_sum_kernel(const float* __restrict__ left, const float* __restrict__ right, const float* __restrict__ left_weight,
                       const float* __restrict__ right_weight, float* __restrict__ out, int width, float eps, float left_scale, float right_scale) {
    grid_dependents_launch();
    grid_dependency_wait();
    __shared__ float scratch[33];
    const size_t base = static_cast<size_t>(blockIdx.x) * width;
    float a = 0.0f, b = 0.0f;
    for (int column = threadIdx.x; column < width; column += blockDim.x) {
        const float x = left[base + column], y = right[base + column];
        a = fmaf(x, x, a);
        b = fmaf(y, y, b);
    }
    const float left_factor = left_scale / sqrtf(block_sum(a, scratch) / static_cast<float>(width) + eps);
    const float right_factor = right_scale / sqrtf(block_sum(b, scratch) / static_cast<float>(width) + eps);
    for (int column = threadIdx.x; column < width; column += blockDim.x)
        out[base + column] = left[base + column] * left_factor * left_weight[column] + right[base + column] * right_factor * right_weight[column];
}

// values [rows, groups * group_width] in 32-bit.  With `normalize` each group of a row is divided by its root mean square;
// then times weight (if any), times sigmoid(gate) or, with `silu_gate`, gate * sigmoid(gate) (if any; gate rows lie `gate_stride`
// apart), rounded once to T; output rows lie `out_stride` apart.
template <typename T>
__global__ void __launch_bounds__(kThreads)
gated_group_norm_kernel(const float* __restrict__ values, const float* __restrict__ weight, const T* __restrict__ gate, long long gate_stride,
                        T* __restrict__ out, long long out_stride, int groups, int group_width, float eps, int normalize, int silu_gate) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int width = groups * group_width;
    const float* source = values + static_cast<size_t>(row) * width;
    __shared__ float scratch[33];
    if (groups >= warps) {       // many groups: a warp takes a group at a time
        for (int group = warp; group < groups; group += warps) {
            float inverse = 1.0f;
            if (normalize) {
                float squares = 0.0f;
                for (int column = lane; column < group_width; column += 32) {
                    const float value = source[group * group_width + column];
                    squares += value * value;
                }
                inverse = 1.0f / sqrtf(warp_sum(squares) / static_cast<float>(group_width) + eps);
            }
            for (int column = lane; column < group_width; column += 32) {
                const int index = group * group_width + column;
                float value = source[index] * inverse;
                if (weight) value *= weight[index];
                if (gate) {
                    const float z = to_float(gate[static_cast<size_t>(row) * gate_stride + index]);
                    value *= (silu_gate ? z : 1.0f) / (1.0f + expf(-z));
                }
                out[static_cast<size_t>(row) * out_stride + index] = from_float<T>(value);
            }
        }
        return;
    }
    for (int group = 0; group < groups; ++group) {     // few groups: the whole block takes one after the other
        float inverse = 1.0f;
        if (normalize) {
            float squares = 0.0f;
            for (int column = threadIdx.x; column < group_width; column += blockDim.x) {
                const float value = source[group * group_width + column];
                squares += value * value;
            }
            inverse = 1.0f / sqrtf(block_sum(squares, scratch) / static_cast<float>(group_width) + eps);
        }
        for (int column = threadIdx.x; column < group_width; column += blockDim.x) {
            const int index = group * group_width + column;
            float value = source[index] * inverse;
            if (weight) value *= weight[index];
            if (gate) {
                const float z = to_float(gate[static_cast<size_t>(row) * gate_stride + index]);
                value *= (silu_gate ? z : 1.0f) / (1.0f + expf(-z));
            }
            out[static_cast<size_t>(row) * out_stride + index] = from_float<T>(value);
        }
    }
}

}  // namespace

TAU_EXPORT int tau_embedding_f32(int table_dtype, const int* tokens, const void* table, float* out, int rows, int width, int vocab, float scale, void* stream) {
    if (rows <= 0) return 0;
    if (!tokens || !table || !out || width <= 0 || vocab <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (table_dtype == TAU_F32) tau_launch(embedding_f32_kernel<float>, dim3(rows), dim3(kThreads), 0, s, tokens, static_cast<const float*>(table), out, width, vocab, scale);
    else if (table_dtype == TAU_BF16) tau_launch(embedding_f32_kernel<bf16>, dim3(rows), dim3(kThreads), 0, s, tokens, static_cast<const bf16*>(table), out, width, vocab, scale);
    else return cudaErrorInvalidValue;
    return tau_launch_status();
}

TAU_EXPORT int tau_stream_add_norm(int out_dtype, float* stream_values, const void* a, int a_dtype, const void* b, int b_dtype, const int* rows,
                                   const float* weight, void* out, int out_rows, int width, float eps, int update, int groups, float branch_scale,
                                   void* stream) {
    if (out_rows <= 0) return 0;
    if (!stream_values || !weight || !out || width <= 0 || (b && !a) || (update && rows) || groups < 1 || groups > kMaxNormGroups || width % groups != 0)
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (out_dtype == TAU_F32) tau_launch(stream_add_norm_kernel<float>, dim3(out_rows), dim3(kThreads), 0, s, stream_values, a, a_dtype, b, b_dtype, rows, weight, static_cast<float*>(out), width, eps, update, groups, branch_scale);
    else if (out_dtype == TAU_BF16) tau_launch(stream_add_norm_kernel<bf16>, dim3(out_rows), dim3(kThreads), 0, s, stream_values, a, a_dtype, b, b_dtype, rows, weight, static_cast<bf16*>(out), width, eps, update, groups, branch_scale);
    else return cudaErrorInvalidValue;
    return tau_launch_status();
}

TAU_EXPORT int tau_normed_pair_sum(const float* left, const float* right, const float* left_weight, const float* right_weight, float* out, int rows, int width,
                                   float eps, float left_scale, float right_scale, void* stream) {
    if (rows <= 0) return 0;
    if (!left || !right || !left_weight || !right_weight || !out || width <= 0) return cudaErrorInvalidValue;
    tau_launch(normed_pair_sum_kernel, dim3(rows), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), left, right, left_weight, right_weight, out, width, eps,
               left_scale, right_scale);
    return tau_launch_status();
}

TAU_EXPORT int tau_gated_group_norm(int dtype, const float* values, const float* weight, const void* gate, long long gate_stride, void* out, long long out_stride,
                                    int rows, int groups, int group_width, float eps, int normalize, int silu_gate, void* stream) {
    if (rows <= 0) return 0;
    if (!values || !out || groups <= 0 || group_width <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int threads = 256;
    if (dtype == TAU_F32) tau_launch(gated_group_norm_kernel<float>, dim3(rows), dim3(threads), 0, s, values, weight, static_cast<const float*>(gate), gate_stride, static_cast<float*>(out), out_stride, groups, group_width, eps, normalize, silu_gate);
    else if (dtype == TAU_BF16) tau_launch(gated_group_norm_kernel<bf16>, dim3(rows), dim3(threads), 0, s, values, weight, static_cast<const bf16*>(gate), gate_stride, static_cast<bf16*>(out), out_stride, groups, group_width, eps, normalize, silu_gate);
    else return cudaErrorInvalidValue;
    return tau_launch_status();
}
