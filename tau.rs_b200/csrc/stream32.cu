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

// r = rows ? rows[i] : i.  sum = stream[r] + (a[r] + b[r]) in 32-bit; if `update` the sum replaces stream[r];
// out[i] = sum / sqrt(mean(sum^2) + eps) * weight, rounded once to T.
template <typename T>
__global__ void __launch_bounds__(kThreads)
stream_add_norm_kernel(float* __restrict__ stream, const void* __restrict__ a, int a_code, const void* __restrict__ b, int b_code,
                       const int* __restrict__ rows, const float* __restrict__ weight, T* __restrict__ out, int width, float eps, int update) {
    grid_dependents_launch();
    grid_dependency_wait();
    __shared__ float scratch[33];
    const int row = rows ? rows[blockIdx.x] : blockIdx.x;
    const size_t base = static_cast<size_t>(row) * width;
    float squares = 0.0f;
    for (int column = threadIdx.x; column < width; column += blockDim.x) {
        float value = stream[base + column];
        if (a) {
            float branch = load_as_float(a, a_code, base + column);
            if (b) branch += load_as_float(b, b_code, base + column);
            value += branch;
        }
        if (update) stream[base + column] = value;
        squares += value * value;
    }
    const float inverse = 1.0f / sqrtf(block_sum(squares, scratch) / static_cast<float>(width) + eps);
    T* target = out + static_cast<size_t>(blockIdx.x) * width;
    for (int column = threadIdx.x; column < width; column += blockDim.x) {
        float value = stream[base + column];     // each thread reads back what it wrote itself
        if (a && !update) {
            float branch = load_as_float(a, a_code, base + column);
            if (b) branch += load_as_float(b, b_code, base + column);
            value += branch;
        }
        target[column] = from_float<T>(value * inverse * weight[column]);
    }
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
                                   const float* weight, void* out, int out_rows, int width, float eps, int update, void* stream) {
    if (out_rows <= 0) return 0;
    if (!stream_values || !weight || !out || width <= 0 || (b && !a) || (update && rows)) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (out_dtype == TAU_F32) tau_launch(stream_add_norm_kernel<float>, dim3(out_rows), dim3(kThreads), 0, s, stream_values, a, a_dtype, b, b_dtype, rows, weight, static_cast<float*>(out), width, eps, update);
    else if (out_dtype == TAU_BF16) tau_launch(stream_add_norm_kernel<bf16>, dim3(out_rows), dim3(kThreads), 0, s, stream_values, a, a_dtype, b, b_dtype, rows, weight, static_cast<bf16*>(out), width, eps, update);
    else return cudaErrorInvalidValue;
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
