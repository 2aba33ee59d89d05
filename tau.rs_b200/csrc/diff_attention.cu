// Differential attention over cached rows: every head has two softmax maps (each with its own query and key of `dim` elements)
// over the same values of `vdim` elements, combined as a1 - lambda * a2, divided by the root mean square over the head's values,
// scaled, and gated by a sigmoid.
//
// One cached row per position: [kv_heads x (map 1 key | map 2 key) | kv_heads x value], keys normalised and rotated already.
//
//   prepare:    per (head, map): q and k divided by their root mean square over `dim` (eps inside the root), times a weight shared
//               by all heads and maps, the first `rotary` elements turned pair by pair (2i, 2i + 1) by position * inv_freq[i];
//               queries to [tokens, heads, 2, dim], keys and values to the token's row.
//   attention:  a warp per (token, head): 32 keys at a time, a lane scores one key for both maps, then every lane sums its own
//               value columns; running maximum and sum per map; scores, weights and sums in 32-bit.
#include "common.cuh"

namespace {

constexpr int kWarps = 8;
constexpr int kMaxOwned = 16;     // value columns per lane: vdim <= 512
constexpr int kMaxPairs = 256;    // rotated pairs whose sine and cosine a block keeps (more are computed where they are used)

// Sine and cosine of position * inv_freq[i] for the block's token, once for all of its maps.
__device__ __forceinline__ void fill_turns(float2* turns, const float* __restrict__ inv_freq, int rotary, int position) {
    const int pairs = rotary / 2 < kMaxPairs ? rotary / 2 : kMaxPairs;
    for (int pair = threadIdx.x; pair < pairs; pair += blockDim.x) {
        float sine, cosine;
        sincosf(static_cast<float>(position) * inv_freq[pair], &sine, &cosine);
        turns[pair] = make_float2(cosine, sine);
    }
    __syncthreads();
}

__device__ __forceinline__ float2 turn_of(const float2* turns, const float* __restrict__ inv_freq, int pair, int position) {
    if (pair < kMaxPairs) return turns[pair];
    float sine, cosine;
    sincosf(static_cast<float>(position) * inv_freq[pair], &sine, &cosine);
    return make_float2(cosine, sine);
}

__device__ __forceinline__ void store_two(float* target, float a, float b) { *reinterpret_cast<float2*>(target) = make_float2(a, b); }
__device__ __forceinline__ void store_two(bf16* target, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(target) = __floats2bfloat162_rn(a, b); }

__device__ __forceinline__ float sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// grid: tokens; a warp per map.  projected row: [heads * 2 * dim | kv_heads * 2 * dim | kv_heads * vdim | ...].
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
diff_prepare_kernel(const T* __restrict__ projected, long long projected_stride, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                    float eps, const float* __restrict__ inv_freq, int rotary, T* __restrict__ queries, T* __restrict__ rows,
                    const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ page_rows, int page_stride,
                    int page_tokens, int heads, int kv_heads, int dim, int vdim, int write_rows) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int token = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int position = positions[token];
    __shared__ float2 turns[kMaxPairs];
    fill_turns(turns, inv_freq, rotary, position);
    const int row_width = kv_heads * (2 * dim + vdim);
    const T* source_row = projected + static_cast<size_t>(token) * projected_stride;
    T* row = nullptr;
    if (write_rows) {
        const int page = page_rows[static_cast<size_t>(token_seq[token]) * page_stride + position / page_tokens];
        row = rows + (static_cast<size_t>(page) * page_tokens + position % page_tokens) * row_width;
    }
    const int q_maps = heads * 2, maps = q_maps + (write_rows ? kv_heads * 2 : 0);
    for (int map = warp; map < maps; map += kWarps) {
        const bool is_query = map < q_maps;
        const T* source = source_row + static_cast<size_t>(map) * dim;      // the key maps follow the query maps in the projected row
        T* target = is_query ? queries + (static_cast<size_t>(token) * q_maps + map) * dim : row + static_cast<size_t>(map - q_maps) * dim;
        const float* weight = is_query ? q_weight : k_weight;
        float squares = 0.0f;
        for (int column = lane; column < dim; column += 32) {
            const float value = to_float(source[column]);
            squares += value * value;
        }
        const float inverse = 1.0f / sqrtf(warp_sum(squares) / static_cast<float>(dim) + eps);
        for (int pair = lane; 2 * pair < dim; pair += 32) {
            const int first = 2 * pair;
            const bool second = first + 1 < dim;
            float u = to_float(source[first]) * inverse * weight[first];
            float w = second ? to_float(source[first + 1]) * inverse * weight[first + 1] : 0.0f;
            if (first + 1 < rotary) {
                const float2 turn = turn_of(turns, inv_freq, pair, position);
                const float a = u * turn.x - w * turn.y, b = w * turn.x + u * turn.y;
                u = a; w = b;
            }
            target[first] = from_float<T>(u);
            if (second) target[first + 1] = from_float<T>(w);
        }
    }
    if (write_rows) {
        const T* values = source_row + static_cast<size_t>(q_maps + kv_heads * 2) * dim;
        T* target = row + static_cast<size_t>(kv_heads) * 2 * dim;
        for (int column = threadIdx.x; column < kv_heads * vdim; column += blockDim.x) target[column] = values[column];
    }
}

// grid: (tokens, ceil(heads / kWarps)); a warp per head.  Dynamic shared memory: kWarps * 2 * dim floats (the queries).
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
diff_attention_kernel(const T* __restrict__ queries, const T* __restrict__ rows, const T* __restrict__ gate, long long gate_stride, T* __restrict__ out,
                      const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ page_rows, int page_stride,
                      int page_tokens, int heads, int kv_heads, int dim, int vdim, float scale, int window, float lambda, float eps, float post_scale) {
    grid_dependents_launch();
    grid_dependency_wait();
    extern __shared__ float shared[];
    const int token = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * kWarps + warp;
    if (head >= heads) return;
    float* query = shared + static_cast<size_t>(warp) * 2 * dim;
    const T* q_source = queries + (static_cast<size_t>(token) * heads + head) * 2 * dim;
    for (int column = lane; column < 2 * dim; column += 32) query[column] = to_float(q_source[column]);
    __syncwarp();
    const int position = positions[token];
    const int* pages = page_rows + static_cast<size_t>(token_seq[token]) * page_stride;
    const int group = head / (heads / kv_heads);
    const int row_width = kv_heads * (2 * dim + vdim);
    const int key_offset = group * 2 * dim, value_offset = kv_heads * 2 * dim + group * vdim;
    const int first_key = window > 0 && position - window + 1 > 0 ? position - window + 1 : 0;
    float top1 = -INFINITY, top2 = -INFINITY, sum1 = 0.0f, sum2 = 0.0f;
    float acc1[kMaxOwned], acc2[kMaxOwned];
#pragma unroll
    for (int i = 0; i < kMaxOwned; ++i) acc1[i] = acc2[i] = 0.0f;
    for (int base = first_key; base <= position; base += 32) {
        const int key = base + lane;
        const bool valid = key <= position;
        long long row_index = 0;
        float s1 = -INFINITY, s2 = -INFINITY;
        if (valid) {
            row_index = static_cast<long long>(pages[key / page_tokens]) * page_tokens + key % page_tokens;
            const T* k = rows + row_index * row_width + key_offset;
            float a = 0.0f, b = 0.0f;
            for (int column = 0; column < dim; ++column) {
                a = fmaf(query[column], to_float(k[column]), a);
                b = fmaf(query[dim + column], to_float(k[dim + column]), b);
            }
            s1 = a * scale;
            s2 = b * scale;
        }
        const float new1 = fmaxf(top1, warp_max(s1)), new2 = fmaxf(top2, warp_max(s2));     // finite: the block holds at least one key
        const float p1 = valid ? expf(s1 - new1) : 0.0f, p2 = valid ? expf(s2 - new2) : 0.0f;
        const float keep1 = expf(top1 - new1), keep2 = expf(top2 - new2);                    // exp(-inf) = 0 the first time
        sum1 = sum1 * keep1 + warp_sum(p1);
        sum2 = sum2 * keep2 + warp_sum(p2);
        top1 = new1;
        top2 = new2;
#pragma unroll
        for (int i = 0; i < kMaxOwned; ++i) { acc1[i] *= keep1; acc2[i] *= keep2; }
        const int count = position - base + 1 < 32 ? position - base + 1 : 32;
        for (int j = 0; j < count; ++j) {
            const float w1 = __shfl_sync(0xffffffffu, p1, j), w2 = __shfl_sync(0xffffffffu, p2, j);
            const long long index = __shfl_sync(0xffffffffu, row_index, j);
            const T* v = rows + index * row_width + value_offset;
#pragma unroll
            for (int i = 0; i < kMaxOwned; ++i) {
                const int column = lane + 32 * i;
                if (column < vdim) {
                    const float value = to_float(v[column]);
                    acc1[i] = fmaf(w1, value, acc1[i]);
                    acc2[i] = fmaf(w2, value, acc2[i]);
                }
            }
        }
    }
    float squares = 0.0f;
#pragma unroll
    for (int i = 0; i < kMaxOwned; ++i) {
        acc1[i] = acc1[i] / sum1 - lambda * (acc2[i] / sum2);
        if (lane + 32 * i < vdim) squares += acc1[i] * acc1[i];
    }
    const float inverse = post_scale / sqrtf(warp_sum(squares) / static_cast<float>(vdim) + eps);
#pragma unroll
    for (int i = 0; i < kMaxOwned; ++i) {
        const int column = lane + 32 * i;
        if (column < vdim) {
            float value = acc1[i] * inverse;
            if (gate) value *= sigmoid(to_float(gate[static_cast<size_t>(token) * gate_stride + head * vdim + column]));
            out[(static_cast<size_t>(token) * heads + head) * vdim + column] = from_float<T>(value);
        }
    }
}

// The same preparation for the cache of ordinary heads: every map is a head of its own, `wide` = max(dim, vdim) elements,
// zeros behind what it holds.  Query (head, map) goes to slot (group * 2 + map) * (heads / kv_heads) + head % (heads / kv_heads)
// of queries [tokens, 2 * heads, wide], so that the slots of one key/value head (group, map) lie together; key pages
// [pages, 2 * kv_heads, page_tokens, wide] hold map `map` of group `group` under head group * 2 + map, value pages hold the
// group's values under both.
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
diff_prepare_wide_kernel(const T* __restrict__ projected, long long projected_stride, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                         float eps, const float* __restrict__ inv_freq, int rotary, T* __restrict__ queries, T* __restrict__ key_pages,
                         T* __restrict__ value_pages, const int* __restrict__ positions, const int* __restrict__ token_seq,
                         const int* __restrict__ page_rows, int page_stride, int page_tokens, int heads, int kv_heads, int dim, int vdim, int wide,
                         int write_cache) {
    // grid: (tokens, y); the warps of a token's y blocks share out its items: the query maps, then (with `write_cache`) the key
    // maps, then the value heads.  Few tokens get a warp per item, many tokens one block each.
    grid_dependents_launch();
    grid_dependency_wait();
    const int token = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int position = positions[token];
    __shared__ float2 turns[kMaxPairs];
    fill_turns(turns, inv_freq, rotary, position);
    const int q_maps = heads * 2, maps = q_maps + (write_cache ? kv_heads * 2 : 0), items = maps + (write_cache ? kv_heads * 2 : 0);
    const int per_group = heads / kv_heads;
    const T* source_row = projected + static_cast<size_t>(token) * projected_stride;
    size_t page_base = 0;
    if (write_cache) {
        const int page = page_rows[static_cast<size_t>(token_seq[token]) * page_stride + position / page_tokens];
        page_base = static_cast<size_t>(page) * 2 * kv_heads * page_tokens * wide + static_cast<size_t>(position % page_tokens) * wide;
    }
    const size_t head_pitch = static_cast<size_t>(page_tokens) * wide;
    for (int item = blockIdx.y * kWarps + warp; item < items; item += gridDim.y * kWarps) {
        if (item >= maps) {          // a value head: the group's values, zeros behind them
            const int head = item - maps;
            const T* values = source_row + static_cast<size_t>(q_maps + kv_heads * 2) * dim + static_cast<size_t>(head >> 1) * vdim;
            T* target = value_pages + page_base + static_cast<size_t>(head) * head_pitch;
            for (int column = 2 * lane; column < wide; column += 64)
                store_two(target + column, column < vdim ? to_float(values[column]) : 0.0f, column + 1 < vdim ? to_float(values[column + 1]) : 0.0f);
            continue;
        }
        const int map = item;
        const bool is_query = map < q_maps;
        const T* source = source_row + static_cast<size_t>(map) * dim;
        T* target;
        if (is_query) {
            const int head = map >> 1, which = map & 1;
            const int slot = ((head / per_group) * 2 + which) * per_group + head % per_group;
            target = queries + (static_cast<size_t>(token) * q_maps + slot) * wide;
        } else {
            target = key_pages + page_base + static_cast<size_t>(map - q_maps) * head_pitch;
        }
        const float* weight = is_query ? q_weight : k_weight;
        float squares = 0.0f;
        for (int column = lane; column < dim; column += 32) {
            const float value = to_float(source[column]);
            squares += value * value;
        }
        const float inverse = 1.0f / sqrtf(warp_sum(squares) / static_cast<float>(dim) + eps);
        for (int pair = lane; 2 * pair < wide; pair += 32) {
            const int first = 2 * pair;
            float u = first < dim ? to_float(source[first]) * inverse * weight[first] : 0.0f;
            float w = first + 1 < dim ? to_float(source[first + 1]) * inverse * weight[first + 1] : 0.0f;
            if (first + 1 < rotary) {
                const float2 turn = turn_of(turns, inv_freq, pair, position);
                const float a = u * turn.x - w * turn.y, b = w * turn.x + u * turn.y;
                u = a; w = b;
            }
            store_two(target + first, u, w);        // `wide` is even and every head starts on a multiple of it
        }
    }
}

// grid: tokens; a warp per head.  attended [tokens, 2 * heads, wide] in the slots of the kernel above.  A lane owns runs of V
// neighbouring columns (V = 4 where vdim, wide and the gate's rows allow 8-byte accesses).
template <typename T, int V>
__global__ void __launch_bounds__(kWarps * 32)
diff_combine_kernel(const T* __restrict__ attended, const T* __restrict__ gate, long long gate_stride, T* __restrict__ out, int heads, int kv_heads,
                    int vdim, int wide, float lambda, float eps, float post_scale) {
    grid_dependents_launch();
    grid_dependency_wait();
    constexpr int kRuns = kMaxOwned / V;
    const int token = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, per_group = heads / kv_heads;
    for (int head = warp; head < heads; head += kWarps) {
        const int slot = (head / per_group) * 2 * per_group + head % per_group;
        const T* first = attended + (static_cast<size_t>(token) * 2 * heads + slot) * wide;
        const T* second = first + static_cast<size_t>(per_group) * wide;
        const T* gates = gate ? gate + static_cast<size_t>(token) * gate_stride + head * vdim : nullptr;
        T* target = out + (static_cast<size_t>(token) * heads + head) * vdim;
        float held[kRuns][V];
        float squares = 0.0f;
#pragma unroll
        for (int i = 0; i < kRuns; ++i) {
            const int column = (lane + 32 * i) * V;
            if (column < vdim) {
                __align__(8) T a[V];
                __align__(8) T b[V];
                if constexpr (V == 4) {
                    *reinterpret_cast<uint2*>(a) = *reinterpret_cast<const uint2*>(first + column);      // V == 4 is used for 2-byte types only
                    *reinterpret_cast<uint2*>(b) = *reinterpret_cast<const uint2*>(second + column);
                } else {
                    a[0] = first[column];
                    b[0] = second[column];
                }
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    held[i][e] = to_float(a[e]) - lambda * to_float(b[e]);
                    squares += held[i][e] * held[i][e];
                }
            }
        }
        const float inverse = post_scale / sqrtf(warp_sum(squares) / static_cast<float>(vdim) + eps);
#pragma unroll
        for (int i = 0; i < kRuns; ++i) {
            const int column = (lane + 32 * i) * V;
            if (column < vdim) {
                __align__(8) T g[V];
                __align__(8) T result[V];
                if (gates) {
                    if constexpr (V == 4) *reinterpret_cast<uint2*>(g) = *reinterpret_cast<const uint2*>(gates + column);
                    else g[0] = gates[column];
                }
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    float value = held[i][e] * inverse;
                    if (gates) value *= sigmoid(to_float(g[e]));
                    result[e] = from_float<T>(value);
                }
                if constexpr (V == 4) *reinterpret_cast<uint2*>(target + column) = *reinterpret_cast<const uint2*>(result);
                else target[column] = result[0];
            }
        }
    }
}

}  // namespace

TAU_EXPORT int tau_diff_prepare_wide(int dtype, const void* projected, long long projected_stride, const float* q_weight, const float* k_weight, float eps,
                                     const float* inv_freq, int rotary, void* queries, void* key_pages, void* value_pages, const int* positions,
                                     const int* token_seq, const int* page_rows, int page_stride, int page_tokens, int tokens, int heads, int kv_heads,
                                     int dim, int vdim, int wide, int write_cache, void* stream) {
    if (tokens <= 0) return 0;
    if (!projected || !q_weight || !k_weight || !queries || !positions || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || dim <= 0 || vdim <= 0
        || wide < dim || wide < vdim || (wide & 1) || rotary < 0 || rotary > dim || (rotary & 1) || (rotary > 0 && !inv_freq)
        || (write_cache && (!key_pages || !value_pages || !token_seq || !page_rows)))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int items = heads * 2 + (write_cache ? kv_heads * 4 : 0);
    const dim3 grid(tokens, tokens >= 1024 ? 1 : (items + kWarps - 1) / kWarps);
    if (dtype == TAU_F32)
        tau_launch(diff_prepare_wide_kernel<float>, grid, dim3(kWarps * 32), 0, s, static_cast<const float*>(projected), projected_stride, q_weight,
                   k_weight, eps, inv_freq, rotary, static_cast<float*>(queries), static_cast<float*>(key_pages), static_cast<float*>(value_pages), positions,
                   token_seq, page_rows, page_stride, page_tokens, heads, kv_heads, dim, vdim, wide, write_cache);
    else if (dtype == TAU_BF16)
        tau_launch(diff_prepare_wide_kernel<bf16>, grid, dim3(kWarps * 32), 0, s, static_cast<const bf16*>(projected), projected_stride, q_weight,
                   k_weight, eps, inv_freq, rotary, static_cast<bf16*>(queries), static_cast<bf16*>(key_pages), static_cast<bf16*>(value_pages), positions,
                   token_seq, page_rows, page_stride, page_tokens, heads, kv_heads, dim, vdim, wide, write_cache);
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}

TAU_EXPORT int tau_diff_combine(int dtype, const void* attended, const void* gate, long long gate_stride, void* out, int tokens, int heads, int kv_heads,
                                int vdim, int wide, float lambda, float eps, float post_scale, void* stream) {
    if (tokens <= 0) return 0;
    if (!attended || !out || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || vdim <= 0 || vdim > 32 * kMaxOwned || wide < vdim) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TAU_F32) {
        tau_launch(diff_combine_kernel<float, 1>, dim3(tokens), dim3(kWarps * 32), 0, s, static_cast<const float*>(attended), static_cast<const float*>(gate),
                   gate_stride, static_cast<float*>(out), heads, kv_heads, vdim, wide, lambda, eps, post_scale);
    } else if (dtype == TAU_BF16) {
        const bool four = vdim % 4 == 0 && wide % 4 == 0 && gate_stride % 4 == 0
                          && ((reinterpret_cast<uintptr_t>(attended) | reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(out)) & 7) == 0;
        tau_launch(four ? diff_combine_kernel<bf16, 4> : diff_combine_kernel<bf16, 1>, dim3(tokens), dim3(kWarps * 32), 0, s,
                   static_cast<const bf16*>(attended), static_cast<const bf16*>(gate), gate_stride, static_cast<bf16*>(out), heads, kv_heads, vdim, wide,
                   lambda, eps, post_scale);
    } else {
        return cudaErrorInvalidValue;
    }
    return tau_launch_status();
}

TAU_EXPORT int tau_diff_prepare(int dtype, const void* projected, long long projected_stride, const float* q_weight, const float* k_weight, float eps,
                                const float* inv_freq, int rotary, void* queries, void* rows, const int* positions, const int* token_seq,
                                const int* page_rows, int page_stride, int page_tokens, int tokens, int heads, int kv_heads, int dim, int vdim,
                                int write_rows, void* stream) {
    if (tokens <= 0) return 0;
    if (!projected || !q_weight || !k_weight || !queries || !positions || heads <= 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || rotary < 0 || rotary > dim
        || (rotary & 1) || (rotary > 0 && !inv_freq) || (write_rows && (!rows || !token_seq || !page_rows)))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TAU_F32)
        tau_launch(diff_prepare_kernel<float>, dim3(tokens), dim3(kWarps * 32), 0, s, static_cast<const float*>(projected), projected_stride, q_weight, k_weight,
                   eps, inv_freq, rotary, static_cast<float*>(queries), static_cast<float*>(rows), positions, token_seq, page_rows, page_stride, page_tokens,
                   heads, kv_heads, dim, vdim, write_rows);
    else if (dtype == TAU_BF16)
        tau_launch(diff_prepare_kernel<bf16>, dim3(tokens), dim3(kWarps * 32), 0, s, static_cast<const bf16*>(projected), projected_stride, q_weight, k_weight,
                   eps, inv_freq, rotary, static_cast<bf16*>(queries), static_cast<bf16*>(rows), positions, token_seq, page_rows, page_stride, page_tokens,
                   heads, kv_heads, dim, vdim, write_rows);
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}

TAU_EXPORT int tau_diff_attention(int dtype, const void* queries, const void* rows, const void* gate, long long gate_stride, void* out, const int* positions,
                                  const int* token_seq, const int* page_rows, int page_stride, int page_tokens, int tokens, int heads, int kv_heads,
                                  int dim, int vdim, float scale, int window, float lambda, float eps, float post_scale, void* stream) {
    if (tokens <= 0) return 0;
    if (!queries || !rows || !out || !positions || !token_seq || !page_rows || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || dim <= 0 || vdim <= 0
        || vdim > 32 * kMaxOwned || window < 0)
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t bytes = static_cast<size_t>(kWarps) * 2 * dim * sizeof(float);
    if (bytes > 48 * 1024) return cudaErrorInvalidValue;
    const dim3 grid(tokens, (heads + kWarps - 1) / kWarps), block(kWarps * 32);
    if (dtype == TAU_F32)
        tau_launch(diff_attention_kernel<float>, grid, block, bytes, s, static_cast<const float*>(queries), static_cast<const float*>(rows),
                   static_cast<const float*>(gate), gate_stride, static_cast<float*>(out), positions, token_seq, page_rows, page_stride, page_tokens, heads,
                   kv_heads, dim, vdim, scale, window, lambda, eps, post_scale);
    else if (dtype == TAU_BF16)
        tau_launch(diff_attention_kernel<bf16>, grid, block, bytes, s, static_cast<const bf16*>(queries), static_cast<const bf16*>(rows),
                   static_cast<const bf16*>(gate), gate_stride, static_cast<bf16*>(out), positions, token_seq, page_rows, page_stride, page_tokens, heads,
                   kv_heads, dim, vdim, scale, window, lambda, eps, post_scale);
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}
