// Grouped-query softmax attention over cached rows for heads of any sizes, with the mask and the denominator as parameters:
//
//   * key and value sizes may differ (`dim`, `vdim`); one cached row per position holds [kv_heads x key | kv_heads x value], or keys
//     and values lie in pages of their own in the layout of ordinary heads, [pages, kv_heads, positions of a page, dim or vdim];
//   * a query at position i sees key j <= i if j > i - window (`window` > 0), or if j lies in i's chunk, floor(j / chunk) ==
//     floor(i / chunk) (`chunk` > 0; chunks are counted from position 0 of the sequence), or always (both 0);
//   * `sink`: the denominator of the softmax has exp(0) added (a key with score 0 and no value);
//   * the result is multiplied by `out_scale` before its one rounding; output rows may lie any distance apart;
//   * `distance` (two numbers r1, r2 per head): r1 * ln(1 + r2 * (i - j)) is taken off the score of key j for the query at i;
//   * `sigmoid_weights`: no softmax; a visible key weighs sigmoid(score + head_offset[head]) and the weights are not normalised;
//   * `gate`: the result is multiplied by sigmoid(gate), one number per (token, head) or one per element of the head's result;
//   * prepare may multiply the query at position p by 1 + coef * ln(floor((p + 1) / every) + 1) (a temperature that grows with the
//     position), and may be asked for the queries alone (a layer that reads the keys and values another layer cached).
//
//   prepare:    q and k divided by the root mean square over the WHOLE projection (all heads together; eps inside the root) and
//               multiplied by a weight of that size (or left as they are without weights); then in every head the first `rotary`
//               elements are turned: element i is paired with element i + rotary / 2, by the angle position * frequency[i], with
//               sine and cosine multiplied by `magnitude`; queries to [tokens, heads, dim], keys and values to the token's row.
//   attention:  a warp per (token, head): 32 keys at a time, a lane scores one key, then every lane sums its own value columns;
//               running maximum (never below the sink's 0 when there is one) and sum; scores, weights and sums in 32-bit.
#include "common.cuh"

namespace {

constexpr int kWarps = 8;
constexpr int kMaxOwned = 16;     // value columns per lane: vdim <= 512

// grid: tokens; block kWarps * 32.  projected row: [heads * dim | kv_heads * dim | kv_heads * vdim] from its first column on.
// Dynamic shared memory: rotary / 2 float2 (cosine, sine).
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
masked_prepare_kernel(const T* __restrict__ projected, long long projected_stride, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                      float eps, const float* __restrict__ frequency, int rotary, float magnitude, T* __restrict__ queries, T* __restrict__ rows,
                      T* __restrict__ value_pages, const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ page_rows, int page_stride,
                      int page_tokens, int heads, int kv_heads, int dim, int vdim, int write_rows, float temperature_coef, int temperature_every) {
    grid_dependents_launch();
    grid_dependency_wait();
    extern __shared__ float2 turns[];
    __shared__ float scratch[33];
    const int token = blockIdx.x;
    const int position = positions[token];
    const int half = rotary / 2;
    for (int pair = threadIdx.x; pair < half; pair += blockDim.x) {
        float sine, cosine;
        sincosf(static_cast<float>(position) * frequency[pair], &sine, &cosine);
        turns[pair] = make_float2(cosine * magnitude, sine * magnitude);
    }
    const T* source = projected + static_cast<size_t>(token) * projected_stride;
    const int q_width = heads * dim, k_width = kv_heads * dim;
    float q_inverse = 1.0f, k_inverse = 1.0f;
    if (q_weight) {
        float squares = 0.0f;
        for (int column = threadIdx.x; column < q_width; column += blockDim.x) {
            const float value = to_float(source[column]);
            squares = fmaf(value, value, squares);
        }
        q_inverse = 1.0f / sqrtf(block_sum(squares, scratch) / static_cast<float>(q_width) + eps);
    }
    if (k_weight && write_rows) {
        float squares = 0.0f;
        for (int column = threadIdx.x; column < k_width; column += blockDim.x) {
            const float value = to_float(source[q_width + column]);
            squares = fmaf(value, value, squares);
        }
        k_inverse = 1.0f / sqrtf(block_sum(squares, scratch) / static_cast<float>(k_width) + eps);
    }
    if (temperature_every > 0) q_inverse *= 1.0f + temperature_coef * logf(static_cast<float>((position + 1) / temperature_every + 1));
    __syncthreads();      // the turns are complete
    // Where the token's keys and values go: head `g`'s key at row + g * key_head_stride, its value at value_row + g * value_head_stride.
    T* row = nullptr;
    T* value_row = nullptr;
    size_t key_head_stride = dim, value_head_stride = vdim;
    if (write_rows) {
        const size_t page = page_rows[static_cast<size_t>(token_seq[token]) * page_stride + position / page_tokens];
        const int within_page = position % page_tokens;
        if (value_pages) {      // keys and values in pages of their own, [pages, kv_heads, page_tokens, dim or vdim]
            key_head_stride = static_cast<size_t>(page_tokens) * dim, value_head_stride = static_cast<size_t>(page_tokens) * vdim;
            row = rows + page * kv_heads * key_head_stride + static_cast<size_t>(within_page) * dim;
            value_row = value_pages + page * kv_heads * value_head_stride + static_cast<size_t>(within_page) * vdim;
        } else {
            row = rows + (page * page_tokens + within_page) * (static_cast<size_t>(kv_heads) * (dim + vdim));
            value_row = row + k_width;
        }
    }
    // Items: within each head, the `half` rotated pairs, then the dim - rotary elements that pass.
    const int per_head = half + (dim - rotary);
    const int q_items = heads * per_head, items = q_items + (write_rows ? kv_heads * per_head : 0);
    for (int item = threadIdx.x; item < items; item += blockDim.x) {
        const bool is_query = item < q_items;
        const int index = is_query ? item : item - q_items;
        const int head = index / per_head, within = index % per_head;
        const T* from = source + (is_query ? 0 : q_width) + head * dim;
        const float* weight = is_query ? q_weight : k_weight;
        const float inverse = is_query ? q_inverse : k_inverse;
        T* target = is_query ? queries + static_cast<size_t>(token) * q_width + head * dim : row + head * key_head_stride;
        if (within < half) {
            const int first = within, second = within + half;
            float u = to_float(from[first]) * inverse, w = to_float(from[second]) * inverse;
            if (weight) {
                u *= weight[head * dim + first];
                w *= weight[head * dim + second];
            }
            const float2 turn = turns[within];
            target[first] = from_float<T>(u * turn.x - w * turn.y);
            target[second] = from_float<T>(w * turn.x + u * turn.y);
        } else {
            const int column = rotary + (within - half);
            float u = to_float(from[column]) * inverse;
            if (weight) u *= weight[head * dim + column];
            target[column] = from_float<T>(u);
        }
    }
    if (write_rows) {
        const T* values = source + q_width + k_width;
        for (int column = threadIdx.x; column < kv_heads * vdim; column += blockDim.x) value_row[(column / vdim) * value_head_stride + column % vdim] = values[column];
    }
}

// grid: (tokens, ceil(heads / kWarps)); a warp per head.  Dynamic shared memory: kWarps * dim floats (the queries).
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
masked_attention_kernel(const T* __restrict__ queries, const T* __restrict__ rows, const T* __restrict__ value_pages, T* __restrict__ out, long long out_stride,
                        const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ page_rows, int page_stride,
                        int page_tokens, int heads, int kv_heads, int dim, int vdim, float scale, int window, int chunk, int sink, float out_scale,
                        const float* __restrict__ distance, int sigmoid_weights, const float* __restrict__ head_offset, const T* __restrict__ gate,
                        long long gate_stride, int gate_per_head) {
    grid_dependents_launch();
    grid_dependency_wait();
    extern __shared__ float shared[];
    const int token = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * kWarps + warp;
    if (head >= heads) return;
    float* query = shared + static_cast<size_t>(warp) * dim;
    const T* q_source = queries + (static_cast<size_t>(token) * heads + head) * dim;
    for (int column = lane; column < dim; column += 32) query[column] = to_float(q_source[column]) * scale;
    __syncwarp();
    const int position = positions[token];
    const int* pages = page_rows + static_cast<size_t>(token_seq[token]) * page_stride;
    const int group = head / (heads / kv_heads);
    // Position `r` of page `p`: this head's key at keys + p * key_page + r * key_row, its value at values + p * value_page + r * value_row.
    const T* keys;
    const T* values;
    long long key_page, key_row, value_page, value_row;
    if (value_pages) {      // [pages, kv_heads, page_tokens, dim or vdim]
        key_row = dim, value_row = vdim, key_page = static_cast<long long>(kv_heads) * page_tokens * dim, value_page = static_cast<long long>(kv_heads) * page_tokens * vdim;
        keys = rows + static_cast<long long>(group) * page_tokens * dim, values = value_pages + static_cast<long long>(group) * page_tokens * vdim;
    } else {                // [pages, page_tokens, keys of all heads | values of all heads]
        key_row = value_row = kv_heads * (dim + vdim), key_page = value_page = key_row * page_tokens;
        keys = rows + group * dim, values = rows + kv_heads * dim + group * vdim;
    }
    int first_key = 0;
    if (window > 0 && position - window + 1 > 0) first_key = position - window + 1;
    if (chunk > 0) first_key = position / chunk * chunk;
    float top = sink ? 0.0f : -INFINITY, sum = sink ? 1.0f : 0.0f;       // the sink: a weight of exp(0 - top) that carries no value
    const float far = distance ? distance[2 * head] : 0.0f, reach = distance ? distance[2 * head + 1] : 0.0f;
    const float offset = head_offset ? head_offset[head] : 0.0f;
    float acc[kMaxOwned];
#pragma unroll
    for (int i = 0; i < kMaxOwned; ++i) acc[i] = 0.0f;
    for (int base = first_key; base <= position; base += 32) {
        const int key = base + lane;
        const bool valid = key <= position;
        long long value_index = 0;
        float score = -INFINITY;
        if (valid) {
            const long long page = pages[key / page_tokens], within_page = key % page_tokens;
            value_index = page * value_page + within_page * value_row;
            const T* k = keys + page * key_page + within_page * key_row;
            float a = 0.0f, b = 0.0f;
            int column = 0;
            for (; column + 1 < dim; column += 2) {
                a = fmaf(query[column], to_float(k[column]), a);
                b = fmaf(query[column + 1], to_float(k[column + 1]), b);
            }
            if (column < dim) a = fmaf(query[column], to_float(k[column]), a);
            score = a + b;
            if (distance) score -= far * log1pf(reach * static_cast<float>(position - key));
        }
        float p;
        if (sigmoid_weights) {
            p = valid ? 1.0f / (1.0f + expf(-(score + offset))) : 0.0f;
        } else {
            const float new_top = fmaxf(top, warp_max(score));       // finite: the block holds at least one key
            p = valid ? expf(score - new_top) : 0.0f;
            const float keep = expf(top - new_top);                   // exp(-inf) = 0 the first time without a sink
            sum = sum * keep + warp_sum(p);
            top = new_top;
#pragma unroll
            for (int i = 0; i < kMaxOwned; ++i) acc[i] *= keep;
        }
        const int count = position - base + 1 < 32 ? position - base + 1 : 32;
        for (int j = 0; j < count; ++j) {
            const float w = __shfl_sync(0xffffffffu, p, j);
            const T* v = values + __shfl_sync(0xffffffffu, value_index, j);
#pragma unroll
            for (int i = 0; i < kMaxOwned; ++i) {
                const int column = lane + 32 * i;
                if (column < vdim) acc[i] = fmaf(w, to_float(v[column]), acc[i]);
            }
        }
    }
    const float factor = sigmoid_weights ? out_scale : out_scale / sum;
    const T* gates = gate ? gate + static_cast<size_t>(token) * gate_stride + (gate_per_head ? head : head * vdim) : nullptr;
#pragma unroll
    for (int i = 0; i < kMaxOwned; ++i) {
        const int column = lane + 32 * i;
        if (column < vdim) {
            float value = acc[i] * factor;
            if (gates) value /= 1.0f + expf(-to_float(gates[gate_per_head ? 0 : column]));
            out[static_cast<size_t>(token) * out_stride + head * vdim + column] = from_float<T>(value);
        }
    }
}

// ---- single tokens (and any step whose sizes allow): tiles of keys and values staged in shared memory --------------------------
//
// grid: (tokens, kv_heads * ceil(group / kStagedWarps)); block: kStagedWarps warps, one per query head of the key/value head's group.
// All threads bring tiles of 32 positions into shared memory with cp.async, 4 bytes at a time (rows of the cache lie 4-byte
// aligned because dim and vdim are multiples of a word's elements), two tiles deep, so that the group's heads share one pass over
// the cache and the loads are whole rows.  Key rows are an odd number of words apart: lane j reads key j without bank conflicts.
// Then as above: a lane scores one key, every lane sums its own value columns; maximum, weights and sums in 32-bit.
// With `splits` > 1 the grid's z cuts a token's tiles into that many ranges, a block leaves its range's sums, maximum and denominator
// in `partial` ([tokens, heads, splits, vdim + 2] floats), and `masked_attention_merge_kernel` joins them: few tokens over a long
// context then fill the machine.
constexpr int kStagedWarps = 4;
constexpr int kTileKeys = 32;

__device__ __forceinline__ void copy_word(void* target, const void* source) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(target))), "l"(source) : "memory");
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename T> struct Word;
template <> struct Word<float> {
    static constexpr int kElements = 1;
    static __device__ __forceinline__ float first(uint32_t word) { return __uint_as_float(word); }
    static __device__ __forceinline__ float second(uint32_t) { return 0.0f; }
};
template <> struct Word<bf16> {
    static constexpr int kElements = 2;
    static __device__ __forceinline__ float first(uint32_t word) { return __uint_as_float(word << 16); }
    static __device__ __forceinline__ float second(uint32_t word) { return __uint_as_float(word & 0xffff0000u); }
};

__host__ __device__ inline int key_stride_words(int key_words) { return key_words | 1; }

template <typename T>
__global__ void __launch_bounds__(kStagedWarps * 32)
masked_attention_staged_kernel(const T* __restrict__ queries, const T* __restrict__ rows, const T* __restrict__ value_pages, T* __restrict__ out,
                               long long out_stride, const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ page_rows,
                               int page_stride, int page_tokens, int heads, int kv_heads, int dim, int vdim, float scale, int window, int chunk, int sink,
                               float out_scale, const float* __restrict__ distance, int sigmoid_weights, const float* __restrict__ head_offset,
                               const T* __restrict__ gate, long long gate_stride, int gate_per_head, int splits, float* __restrict__ partial) {
    grid_dependents_launch();
    grid_dependency_wait();
    constexpr int kPer = Word<T>::kElements;
    extern __shared__ __align__(16) uint32_t staged_words[];
    const int key_words = dim / kPer, value_words = vdim / kPer, key_stride = key_stride_words(key_words);
    const int tile_words = kTileKeys * (key_stride + value_words);
    float* query_rows = reinterpret_cast<float*>(staged_words + 2 * tile_words);       // [kStagedWarps][dim]
    const int token = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group_size = heads / kv_heads, passes = (group_size + kStagedWarps - 1) / kStagedWarps;
    const int group = blockIdx.y / passes, head_in_group = (blockIdx.y % passes) * kStagedWarps + warp;
    const bool has_head = head_in_group < group_size;
    const int head = group * group_size + (has_head ? head_in_group : 0);
    const int position = positions[token];
    const int* pages = page_rows + static_cast<size_t>(token_seq[token]) * page_stride;
    const T* keys;
    const T* values;
    long long key_page, key_row, value_page, value_row;
    if (value_pages) {
        key_row = dim, value_row = vdim, key_page = static_cast<long long>(kv_heads) * page_tokens * dim, value_page = static_cast<long long>(kv_heads) * page_tokens * vdim;
        keys = rows + static_cast<long long>(group) * page_tokens * dim, values = value_pages + static_cast<long long>(group) * page_tokens * vdim;
    } else {
        key_row = value_row = kv_heads * (dim + vdim), key_page = value_page = key_row * page_tokens;
        keys = rows + group * dim, values = rows + kv_heads * dim + group * vdim;
    }
    int first_key = 0;
    if (window > 0 && position - window + 1 > 0) first_key = position - window + 1;
    if (chunk > 0) first_key = position / chunk * chunk;
    const int all_tiles = (position - first_key) / kTileKeys + 1;
    // This block's range of the token's tiles (all of them without splits); tiles are numbered from the range's first.
    const int per_split = (all_tiles + splits - 1) / splits, tile_begin = static_cast<int>(blockIdx.z) * per_split;
    const int n_tiles = all_tiles - tile_begin < per_split ? (all_tiles - tile_begin > 0 ? all_tiles - tile_begin : 0) : per_split;
    first_key += tile_begin * kTileKeys;

    auto stage = [&](int tile) {
        uint32_t* buffer = staged_words + (tile & 1) * tile_words;
        if (tile < n_tiles) {
            const int base = first_key + tile * kTileKeys;
            const int count = position - base + 1 < kTileKeys ? position - base + 1 : kTileKeys;
            uint32_t* value_buffer = buffer + kTileKeys * key_stride;
            for (int row = warp; row < count; row += kStagedWarps) {      // a warp per row: one page lookup, then whole lines
                const int key = base + row;
                const long long page = pages[key / page_tokens], within_page = key % page_tokens;
                const uint32_t* key_source = reinterpret_cast<const uint32_t*>(keys + page * key_page + within_page * key_row);
                const uint32_t* value_source = reinterpret_cast<const uint32_t*>(values + page * value_page + within_page * value_row);
                for (int word = lane; word < key_words; word += 32) copy_word(buffer + row * key_stride + word, key_source + word);
                for (int word = lane; word < value_words; word += 32) copy_word(value_buffer + row * value_words + word, value_source + word);
            }
        }
        copy_commit();
    };
    stage(0);
    stage(1);
    if (has_head)
        for (int column = lane; column < dim; column += 32)
            query_rows[warp * dim + column] = to_float(queries[(static_cast<size_t>(token) * heads + head) * dim + column]) * scale;
    const float* query = query_rows + warp * dim;
    const float far = distance ? distance[2 * head] : 0.0f, reach = distance ? distance[2 * head + 1] : 0.0f;
    const float offset = head_offset ? head_offset[head] : 0.0f;
    const bool with_sink = sink && blockIdx.z == 0;      // the added one is counted once
    float top = with_sink ? 0.0f : -INFINITY, sum = with_sink ? 1.0f : 0.0f;
    float acc[kMaxOwned];
#pragma unroll
    for (int i = 0; i < kMaxOwned; ++i) acc[i] = 0.0f;
    for (int tile = 0; tile < n_tiles; ++tile) {
        copy_wait<1>();      // this thread's copies of `tile` are done (those of the next tile may be on their way)
        __syncthreads();     // everybody's are; the queries too
        const uint32_t* buffer = staged_words + (tile & 1) * tile_words;
        const int base = first_key + tile * kTileKeys;
        const int count = position - base + 1 < kTileKeys ? position - base + 1 : kTileKeys;
        if (has_head) {
            float score = -INFINITY;
            if (lane < count) {
                const uint32_t* k = buffer + lane * key_stride;
                float a = 0.0f, b = 0.0f;
                for (int word = 0; word < key_words; ++word) {
                    const uint32_t both = k[word];
                    a = fmaf(query[word * kPer], Word<T>::first(both), a);
                    if (kPer == 2) b = fmaf(query[word * kPer + 1], Word<T>::second(both), b);
                }
                score = a + b;
                if (distance) score -= far * log1pf(reach * static_cast<float>(position - (base + lane)));
            }
            float p;
            if (sigmoid_weights) {
                p = lane < count ? 1.0f / (1.0f + expf(-(score + offset))) : 0.0f;
            } else {
                const float new_top = fmaxf(top, warp_max(score));
                p = lane < count ? expf(score - new_top) : 0.0f;
                const float keep = expf(top - new_top);
                sum = sum * keep + warp_sum(p);
                top = new_top;
#pragma unroll
                for (int i = 0; i < kMaxOwned; ++i) acc[i] *= keep;
            }
            const uint32_t* v = buffer + kTileKeys * key_stride;
            for (int j = 0; j < count; ++j) {
                const float w = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
                for (int i = 0; i < kMaxOwned / kPer; ++i) {
                    const int word = lane + 32 * i;
                    if (word < value_words) {
                        const uint32_t both = v[j * value_words + word];
                        acc[i * kPer] = fmaf(w, Word<T>::first(both), acc[i * kPer]);
                        if (kPer == 2) acc[i * kPer + 1] = fmaf(w, Word<T>::second(both), acc[i * kPer + 1]);
                    }
                }
            }
        }
        __syncthreads();     // the tile's place may be written over
        stage(tile + 2);
    }
    copy_wait<0>();
    if (!has_head) return;
    if (partial) {      // this range's sums as they stand (in the scale of its own maximum), then the maximum and the denominator
        float* record = partial + ((static_cast<size_t>(token) * heads + head) * splits + blockIdx.z) * (vdim + 2);
#pragma unroll
        for (int i = 0; i < kMaxOwned / kPer; ++i) {
            const int word = lane + 32 * i;
            if (word < value_words) {
#pragma unroll
                for (int e = 0; e < kPer; ++e) record[word * kPer + e] = acc[i * kPer + e];
            }
        }
        if (lane == 0) record[vdim] = top, record[vdim + 1] = sum;
        return;
    }
    const float factor = sigmoid_weights ? out_scale : out_scale / sum;
    T* target = out + static_cast<size_t>(token) * out_stride + head * vdim;
    const T* gates = gate ? gate + static_cast<size_t>(token) * gate_stride + (gate_per_head ? head : head * vdim) : nullptr;
#pragma unroll
    for (int i = 0; i < kMaxOwned / kPer; ++i) {
        const int word = lane + 32 * i;
        if (word < value_words) {
#pragma unroll
            for (int e = 0; e < kPer; ++e) {
                float value = acc[i * kPer + e] * factor;
                if (gates) value /= 1.0f + expf(-to_float(gates[gate_per_head ? 0 : word * kPer + e]));
                target[word * kPer + e] = from_float<T>(value);
            }
        }
    }
}

// grid (tokens, heads); block 128.  Joins the ranges that the staged kernel left in `partial`: the sums are brought to the largest
// maximum and added, divided by the joined denominator (sigmoid weights: added as they are), gated and rounded once.
template <typename T>
__global__ void __launch_bounds__(128)
masked_attention_merge_kernel(const float* __restrict__ partial, T* __restrict__ out, long long out_stride, int heads, int vdim, int splits, float out_scale,
                              int sigmoid_weights, const T* __restrict__ gate, long long gate_stride, int gate_per_head) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int token = blockIdx.x, head = blockIdx.y;
    const float* records = partial + (static_cast<size_t>(token) * heads + head) * splits * (vdim + 2);
    float top = -INFINITY;
    if (!sigmoid_weights)
        for (int split = 0; split < splits; ++split) top = fmaxf(top, records[static_cast<size_t>(split) * (vdim + 2) + vdim]);
    float total = 0.0f;
    if (!sigmoid_weights)
        for (int split = 0; split < splits; ++split)
            total += records[static_cast<size_t>(split) * (vdim + 2) + vdim + 1] * expf(records[static_cast<size_t>(split) * (vdim + 2) + vdim] - top);
    const float factor = sigmoid_weights ? out_scale : out_scale / total;
    const T* gates = gate ? gate + static_cast<size_t>(token) * gate_stride + (gate_per_head ? head : head * vdim) : nullptr;
    for (int column = threadIdx.x; column < vdim; column += blockDim.x) {
        float sum = 0.0f;
        for (int split = 0; split < splits; ++split) {
            const float* record = records + static_cast<size_t>(split) * (vdim + 2);
            sum += sigmoid_weights ? record[column] : record[column] * expf(record[vdim] - top);      // a range without keys: exp(-inf) = 0
        }
        float value = sum * factor;
        if (gates) value /= 1.0f + expf(-to_float(gates[gate_per_head ? 0 : column]));
        out[static_cast<size_t>(token) * out_stride + head * vdim + column] = from_float<T>(value);
    }
}

// Shared memory of the staged kernel, or 0 where it does not serve these sizes.
template <typename T>
int staged_bytes(int dim, int vdim) {
    constexpr int kPer = Word<T>::kElements;
    if (dim % kPer != 0 || vdim % kPer != 0) return 0;
    const long long bytes = (2LL * kTileKeys * (key_stride_words(dim / kPer) + vdim / kPer) + static_cast<long long>(kStagedWarps) * dim) * 4;
    return bytes <= 160 * 1024 ? static_cast<int>(bytes) : 0;
}

template <typename T>
int launch_staged(int bytes, const void* queries, const void* rows, const void* value_pages, void* out, long long out_stride, const int* positions,
                  const int* token_seq, const int* page_rows, int page_stride, int page_tokens, int tokens, int heads, int kv_heads, int dim, int vdim,
                  float scale, int window, int chunk, int sink, float out_scale, const float* distance, int sigmoid_weights, const float* head_offset,
                  const void* gate, long long gate_stride, int gate_per_head, int splits, float* partial, cudaStream_t s) {
    static int allowed = 48 * 1024;
    if (bytes > allowed) {
        cudaError_t status = cudaFuncSetAttribute(masked_attention_staged_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        if (status != cudaSuccess) return static_cast<int>(status);
        allowed = 160 * 1024;
    }
    const int group_size = heads / kv_heads, passes = (group_size + kStagedWarps - 1) / kStagedWarps;
    if (splits > 1 && !partial) return cudaErrorInvalidValue;
    if (splits <= 1) splits = 1, partial = nullptr;
    tau_launch(masked_attention_staged_kernel<T>, dim3(tokens, kv_heads * passes, splits), dim3(kStagedWarps * 32), bytes, s, static_cast<const T*>(queries),
               static_cast<const T*>(rows), static_cast<const T*>(value_pages), static_cast<T*>(out), out_stride, positions, token_seq, page_rows, page_stride,
               page_tokens, heads, kv_heads, dim, vdim, scale, window, chunk, sink, out_scale, distance, sigmoid_weights, head_offset,
               static_cast<const T*>(gate), gate_stride, gate_per_head, splits, partial);
    int status = tau_launch_status();
    if (status != 0 || !partial) return status;
    tau_launch(masked_attention_merge_kernel<T>, dim3(tokens, heads), dim3(128), 0, s, partial, static_cast<T*>(out), out_stride, heads, vdim, splits, out_scale,
               sigmoid_weights, static_cast<const T*>(gate), gate_stride, gate_per_head);
    return tau_launch_status();
}

// out[r, c] = values[r, c] * sigmoid(gate[r, c]); rows of the three any distance apart, `out` may be `values`.
template <typename T>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(const T* __restrict__ values, long long values_stride, const T* __restrict__ gate, long long gate_stride, T* __restrict__ out,
                    long long out_stride, int width) {
    grid_dependents_launch();
    grid_dependency_wait();
    const size_t row = blockIdx.x;
    for (int column = threadIdx.x; column < width; column += blockDim.x)
        out[row * out_stride + column] = from_float<T>(to_float(values[row * values_stride + column]) / (1.0f + expf(-to_float(gate[row * gate_stride + column]))));
}

}  // namespace

TAU_EXPORT int tau_sigmoid_gate(int dtype, const void* values, long long values_stride, const void* gate, long long gate_stride, void* out, long long out_stride,
                                int rows, int width, void* stream) {
    if (rows <= 0) return 0;
    if (!values || !gate || !out || width <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TAU_F32)
        tau_launch(sigmoid_gate_kernel<float>, dim3(rows), dim3(256), 0, s, static_cast<const float*>(values), values_stride, static_cast<const float*>(gate), gate_stride,
                   static_cast<float*>(out), out_stride, width);
    else if (dtype == TAU_BF16)
        tau_launch(sigmoid_gate_kernel<bf16>, dim3(rows), dim3(256), 0, s, static_cast<const bf16*>(values), values_stride, static_cast<const bf16*>(gate), gate_stride,
                   static_cast<bf16*>(out), out_stride, width);
    else return cudaErrorInvalidValue;
    return tau_launch_status();
}

TAU_EXPORT int tau_masked_prepare(int dtype, const void* projected, long long projected_stride, const float* q_weight, const float* k_weight, float eps,
                                  const float* frequency, int rotary, float magnitude, void* queries, void* rows, void* value_pages, const int* positions,
                                  const int* token_seq, const int* page_rows, int page_stride, int page_tokens, int tokens, int heads, int kv_heads, int dim, int vdim,
                                  int write_rows, float temperature_coef, int temperature_every, void* stream) {
    if (tokens <= 0) return 0;
    if (!projected || !queries || !positions || heads <= 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || rotary < 0 || rotary > dim || rotary % 2 != 0 ||
        (rotary && !frequency) || (write_rows && (!rows || !token_seq || !page_rows)))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t bytes = static_cast<size_t>(rotary / 2) * sizeof(float2);
    if (bytes > 40 * 1024) return cudaErrorInvalidValue;
#define TAU_PREPARE(T)                                                                                                                            \
    tau_launch(masked_prepare_kernel<T>, dim3(tokens), dim3(kWarps * 32), bytes, s, static_cast<const T*>(projected), projected_stride, q_weight, k_weight, eps, \
               frequency, rotary, magnitude, static_cast<T*>(queries), static_cast<T*>(rows), static_cast<T*>(value_pages), positions, token_seq, page_rows, page_stride, page_tokens, heads,   \
               kv_heads, dim, vdim, write_rows, temperature_coef, temperature_every)
    if (dtype == TAU_F32) TAU_PREPARE(float);
    else if (dtype == TAU_BF16) TAU_PREPARE(bf16);
    else return cudaErrorInvalidValue;
#undef TAU_PREPARE
    return tau_launch_status();
}

// `value_pages` null: `rows` holds one row per position, [pages, page_tokens, kv_heads * (dim + vdim)].  Else keys and values lie in pages
// of their own, `rows` [pages, kv_heads, page_tokens, dim] and `value_pages` [pages, kv_heads, page_tokens, vdim].
TAU_EXPORT int tau_masked_attention(int dtype, const void* queries, const void* rows, const void* value_pages, void* out, long long out_stride, const int* positions,
                                    const int* token_seq, const int* page_rows, int page_stride, int page_tokens, int tokens, int heads, int kv_heads,
                                    int dim, int vdim, float scale, int window, int chunk, int sink, float out_scale, int staged, const float* distance,
                                    int sigmoid_weights, const float* head_offset, const void* gate, long long gate_stride, int gate_per_head, int splits,
                                    float* partial, void* stream) {
    if (tokens <= 0) return 0;
    if (!queries || !rows || !out || !positions || !token_seq || !page_rows || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || dim <= 0 ||
        vdim <= 0 || vdim > 32 * kMaxOwned || window < 0 || chunk < 0 || (window > 0 && chunk > 0) || (sigmoid_weights && sink))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // `staged` (steps of single tokens): the kernel that shares tiles of the cache among a group's heads, where the sizes allow it.
    if (staged && (dtype == TAU_F32 || dtype == TAU_BF16)) {
        const int staged_size = dtype == TAU_F32 ? staged_bytes<float>(dim, vdim) : staged_bytes<bf16>(dim, vdim);
        if (staged_size > 0) {
            if (dtype == TAU_F32)
                return launch_staged<float>(staged_size, queries, rows, value_pages, out, out_stride, positions, token_seq, page_rows, page_stride, page_tokens,
                                            tokens, heads, kv_heads, dim, vdim, scale, window, chunk, sink, out_scale, distance, sigmoid_weights, head_offset, gate, gate_stride,
                                            gate_per_head, splits, partial, s);
            return launch_staged<bf16>(staged_size, queries, rows, value_pages, out, out_stride, positions, token_seq, page_rows, page_stride, page_tokens,
                                       tokens, heads, kv_heads, dim, vdim, scale, window, chunk, sink, out_scale, distance, sigmoid_weights, head_offset, gate, gate_stride,
                                       gate_per_head, splits, partial, s);
        }
    }
    const size_t bytes = static_cast<size_t>(kWarps) * dim * sizeof(float);
    if (bytes > 40 * 1024) return cudaErrorInvalidValue;
    dim3 grid(tokens, (heads + kWarps - 1) / kWarps);
#define TAU_ATTEND(T)                                                                                                                         \
    tau_launch(masked_attention_kernel<T>, grid, dim3(kWarps * 32), bytes, s, static_cast<const T*>(queries), static_cast<const T*>(rows), static_cast<const T*>(value_pages), static_cast<T*>(out), \
               out_stride, positions, token_seq, page_rows, page_stride, page_tokens, heads, kv_heads, dim, vdim, scale, window, chunk, sink, out_scale, distance,         \
               sigmoid_weights, head_offset, static_cast<const T*>(gate), gate_stride, gate_per_head)
    if (dtype == TAU_F32) TAU_ATTEND(float);
    else if (dtype == TAU_BF16) TAU_ATTEND(bf16);
    else return cudaErrorInvalidValue;
#undef TAU_ATTEND
    return tau_launch_status();
}
