// Attention over a cached latent: every position keeps one row [latent (rank) | rotated key part (rot)], shared by all
// heads.  A head's query is [its unrotated part carried into the latent's space (rank) | its rotated part (rot)], so a
// score is one dot product of `rank + rot` elements with the cached row, and the head's output is the weighted sum of
// the rows' latent parts (expanded to values afterwards, by a product per head).
//
//   prepare: latent = RMSnorm(first `rank` elements of the down-projection) * w; the last `rot` elements and every
//            head's rotated query part are rotated at the token's position: the pair (2i, 2i+1), i < rotary/2, by the
//            angle p * inv_freq[i]; the row goes to its cache page, the rotated query parts to the query rows.
//   attend:  causal softmax over the rows of the token's sequence (optionally the last `window` only), scores and
//            weights in 32-bit; a head may have a sink: exp(sink) joins the denominator with no row behind it.
#include "common.cuh"

namespace {

constexpr int kTile = 32;          // cached positions per tile: one per lane
constexpr int kMaxWarps = 8;       // heads per block
constexpr int kMaxOwned = 32;      // latent columns per lane: rank <= 1024

// One block per token.
template <typename T>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const T* __restrict__ down, long long down_stride, const float* __restrict__ latent_weight, float eps,
                      const T* __restrict__ q, long long q_stride, T* __restrict__ queries, T* __restrict__ rows,
                      const float* __restrict__ inv_freq, int rotary, const int* __restrict__ positions, const int* __restrict__ token_seq,
                      const int* __restrict__ page_rows, int page_stride, int page_tokens, int heads, int head_dim, int rot, int rank, int write_rows,
                      T* __restrict__ latent_out) {
    grid_dependents_launch();
    grid_dependency_wait();
    __shared__ float scratch[33];
    const int token = blockIdx.x, position = positions[token];
    const int width = rank + rot;
    if (write_rows) {
        const T* source = down + static_cast<size_t>(token) * down_stride;
        const int page = page_rows[static_cast<size_t>(token_seq[token]) * page_stride + position / page_tokens];
        T* target = rows + (static_cast<size_t>(page) * page_tokens + position % page_tokens) * width;
        float squares = 0.0f;
        for (int column = threadIdx.x; column < rank; column += blockDim.x) {
            const float value = to_float(source[column]);
            squares += value * value;
        }
        const float inverse = 1.0f / sqrtf(block_sum(squares, scratch) / static_cast<float>(rank) + eps);
        for (int column = threadIdx.x; column < rank; column += blockDim.x) {
            const T latent = from_float<T>(to_float(source[column]) * inverse * latent_weight[column]);
            target[column] = latent;
            if (latent_out) latent_out[static_cast<size_t>(token) * rank + column] = latent;     // the same values side by side, for products
        }
        for (int pair = threadIdx.x; pair < rot / 2 + (rot & 1); pair += blockDim.x) {
            const int first = 2 * pair;
            float u = to_float(source[rank + first]), w = first + 1 < rot ? to_float(source[rank + first + 1]) : 0.0f;
            if (first + 1 < rotary) {
                float sine, cosine;
                sincosf(static_cast<float>(position) * inv_freq[pair], &sine, &cosine);
                const float a = u * cosine - w * sine, b = w * cosine + u * sine;
                u = a; w = b;
            }
            target[rank + first] = from_float<T>(u);
            if (first + 1 < rot) target[rank + first + 1] = from_float<T>(w);
        }
    }
    if (!queries) return;
    const int pairs = rot / 2 + (rot & 1);
    for (int item = threadIdx.x; item < heads * pairs; item += blockDim.x) {
        const int head = item / pairs, first = 2 * (item % pairs);
        const T* source = q + static_cast<size_t>(token) * q_stride + head * (head_dim + rot) + head_dim;
        T* target = queries + (static_cast<size_t>(token) * heads + head) * width + rank;
        float u = to_float(source[first]), w = first + 1 < rot ? to_float(source[first + 1]) : 0.0f;
        if (first + 1 < rotary) {
            float sine, cosine;
            sincosf(static_cast<float>(position) * inv_freq[first / 2], &sine, &cosine);
            const float a = u * cosine - w * sine, b = w * cosine + u * sine;
            u = a; w = b;
        }
        target[first] = from_float<T>(u);
        if (first + 1 < rot) target[first + 1] = from_float<T>(w);
    }
}

// One block per (token, group of up to 8 heads); a warp per head.  Tiles of 32 cached rows pass through shared memory
// as floats; lane j scores row j, then every lane accumulates its own latent columns.
template <typename T>
__global__ void __launch_bounds__(kMaxWarps * 32)
latent_attention_kernel(const T* __restrict__ queries, const T* __restrict__ rows, T* __restrict__ out, const float* __restrict__ sinks,
                        const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ page_rows, int page_stride,
                        int page_tokens, int heads, int rank, int rot, float scale, int window) {
    grid_dependents_launch();
    grid_dependency_wait();
    extern __shared__ float shared[];
    const int width = rank + rot, pitch = width + 1;
    float* tile = shared;                                   // [kTile][pitch]
    float* query = shared + kTile * pitch;                  // [warps][width]
    const int token = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * kMaxWarps + warp;
    const bool active = head < heads;
    const int position = positions[token];
    const int* pages = page_rows + static_cast<size_t>(token_seq[token]) * page_stride;
    if (active)
        for (int column = lane; column < width; column += 32)
            query[warp * width + column] = to_float(queries[(static_cast<size_t>(token) * heads + head) * width + column]);
    const int first = window > 0 ? max(0, position - window + 1) : 0;
    float top = -INFINITY, denominator = 0.0f;
    float sums[kMaxOwned];
#pragma unroll
    for (int i = 0; i < kMaxOwned; ++i) sums[i] = 0.0f;
    for (int start = first / kTile * kTile; start <= position; start += kTile) {
        __syncthreads();                                    // the tile before this one has been used up (and the queries are written)
        for (int item = threadIdx.x; item < kTile * width; item += blockDim.x) {
            const int r = item / width, column = item % width, key = start + r;
            float value = 0.0f;
            if (key <= position && key >= first)
                value = to_float(rows[(static_cast<size_t>(pages[key / page_tokens]) * page_tokens + key % page_tokens) * width + column]);
            tile[r * pitch + column] = value;
        }
        __syncthreads();
        if (!active) continue;
        const int key = start + lane;
        float score = -INFINITY;
        if (key <= position && key >= first) {
            float dot = 0.0f;
            const float* mine = tile + lane * pitch;
            const float* wanted = query + warp * width;
            for (int column = 0; column < width; ++column) dot = fmaf(wanted[column], mine[column], dot);
            score = dot * scale;
        }
        const float tile_top = warp_max(score);             // at least the row at `start` or at `position` is visible
        const float new_top = fmaxf(top, tile_top);
        const float rescale = expf(top - new_top);           // 0 the first time
        const float weight = expf(score - new_top);          // 0 for hidden rows
        denominator = denominator * rescale + warp_sum(weight);
        top = new_top;
#pragma unroll
        for (int i = 0; i < kMaxOwned; ++i) sums[i] *= rescale;
        for (int r = 0; r < kTile; ++r) {
            const float w = __shfl_sync(0xffffffffu, weight, r);
            if (w == 0.0f) continue;
#pragma unroll
            for (int i = 0; i < kMaxOwned; ++i) {
                const int column = lane + 32 * i;
                if (column < rank) sums[i] = fmaf(w, tile[r * pitch + column], sums[i]);
            }
        }
    }
    if (!active) return;
    if (sinks) {
        const float sink = sinks[head];
        const float new_top = fmaxf(top, sink);
        const float rescale = expf(top - new_top);
        denominator = denominator * rescale + expf(sink - new_top);
#pragma unroll
        for (int i = 0; i < kMaxOwned; ++i) sums[i] *= rescale;
    }
    const float inverse = 1.0f / denominator;
#pragma unroll
    for (int i = 0; i < kMaxOwned; ++i) {
        const int column = lane + 32 * i;
        if (column < rank) out[(static_cast<size_t>(token) * heads + head) * rank + column] = from_float<T>(sums[i] * inverse);
    }
}

// The same attention with every cached row read once per head as 16-byte vectors and never staged: lane l of a head's warp
// holds elements [8v, 8v + 8) (4 in 32-bit) of the query for v = l, l + 32, ..., reads the same elements of each row, and keeps
// the weighted sums of exactly those elements, so the row that was read for the score is the row that is summed.  Two rows are
// in flight at a time.  The context may be cut into `splits` ranges (grid.z): a range leaves (top, denominator, sums) in
// `partial` and `latent_merge_kernel` joins them; with one range the warp finishes the head itself.
template <typename T> struct RowVectors;
template <> struct RowVectors<bf16> { static constexpr int n = 8, per_lane = 3; };
template <> struct RowVectors<float> { static constexpr int n = 4, per_lane = 6; };
constexpr int kVectorWidth = 768;      // 32 lanes x per_lane x n elements

template <typename T> __device__ __forceinline__ void unpack_row(const uint4& raw, float (&out)[RowVectors<T>::n]);
template <> __device__ __forceinline__ void unpack_row<bf16>(const uint4& raw, float (&out)[8]) {
    const unsigned words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(words[i] << 16);
        out[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000u);
    }
}
template <> __device__ __forceinline__ void unpack_row<float>(const uint4& raw, float (&out)[4]) {
    out[0] = __uint_as_float(raw.x); out[1] = __uint_as_float(raw.y); out[2] = __uint_as_float(raw.z); out[3] = __uint_as_float(raw.w);
}

// dot += q . a and sums += weight * a for one 16-byte vector of a row, unpacked on the way (rows and queries stay packed in
// registers, which keeps two blocks of eight warps on an SM).
template <typename T> __device__ __forceinline__ float vector_dot(const uint4& q, const uint4& a);
template <> __device__ __forceinline__ float vector_dot<bf16>(const uint4& q, const uint4& a) {
    const unsigned qw[4] = {q.x, q.y, q.z, q.w}, aw[4] = {a.x, a.y, a.z, a.w};
    float dot = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        dot = fmaf(__uint_as_float(qw[i] << 16), __uint_as_float(aw[i] << 16), dot);
        dot = fmaf(__uint_as_float(qw[i] & 0xffff0000u), __uint_as_float(aw[i] & 0xffff0000u), dot);
    }
    return dot;
}
template <> __device__ __forceinline__ float vector_dot<float>(const uint4& q, const uint4& a) {
    return fmaf(__uint_as_float(q.x), __uint_as_float(a.x), fmaf(__uint_as_float(q.y), __uint_as_float(a.y),
           fmaf(__uint_as_float(q.z), __uint_as_float(a.z), __uint_as_float(q.w) * __uint_as_float(a.w))));
}

template <typename T>
__global__ void __launch_bounds__(kMaxWarps * 32, 2)
latent_attention_vec_kernel(const T* __restrict__ queries, const T* __restrict__ rows, T* __restrict__ out, const float* __restrict__ sinks,
                            const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ page_rows, int page_stride,
                            int page_tokens, int heads, int rank, int rot, float scale, int window, int splits, float* __restrict__ partial) {
    grid_dependents_launch();
    grid_dependency_wait();
    constexpr int n = RowVectors<T>::n, kPer = RowVectors<T>::per_lane;
    const int token = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, split = blockIdx.z;
    const int head = blockIdx.y * kMaxWarps + warp;
    if (head >= heads) return;                               // the warps of a block never meet
    const int width = rank + rot, vectors = width / n;
    const int position = positions[token];
    const int* pages = page_rows + static_cast<size_t>(token_seq[token]) * page_stride;
    const int first = window > 0 ? max(0, position - window + 1) : 0;
    const int chunk = (position + 1 - first + splits - 1) / splits;
    const int begin = first + split * chunk, end = min(position + 1, begin + chunk);
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    uint4 q[kPer];
    float sums[kPer][n];
    const T* query = queries + (static_cast<size_t>(token) * heads + head) * width;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
        const int v = lane + 32 * i;
#pragma unroll
        for (int j = 0; j < n; ++j) sums[i][j] = 0.0f;
        q[i] = v < vectors ? *reinterpret_cast<const uint4*>(query + v * n) : zero;
    }
    float top = -INFINITY, denominator = 0.0f;
    int key = begin;
    while (key < end) {
        const int page_index = key / page_tokens;
        const int stop = min(end, (page_index + 1) * page_tokens);
        const T* row = rows + (static_cast<size_t>(pages[page_index]) * page_tokens + (key - page_index * page_tokens)) * width;
        for (; key < stop; key += 2, row += 2 * static_cast<size_t>(width)) {
            const bool pair = key + 1 < stop;
            uint4 a[kPer], b[kPer];
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                const int v = lane + 32 * i;
                a[i] = v < vectors ? *reinterpret_cast<const uint4*>(row + v * n) : zero;
                b[i] = (pair && v < vectors) ? *reinterpret_cast<const uint4*>(row + width + v * n) : zero;
            }
            float dot_a = 0.0f, dot_b = 0.0f;
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                dot_a += vector_dot<T>(q[i], a[i]);
                dot_b += vector_dot<T>(q[i], b[i]);
            }
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1) {
                dot_a += __shfl_xor_sync(0xffffffffu, dot_a, offset);
                dot_b += __shfl_xor_sync(0xffffffffu, dot_b, offset);
            }
            dot_a *= scale;
            dot_b *= scale;
            const float new_top = pair ? fmaxf(top, fmaxf(dot_a, dot_b)) : fmaxf(top, dot_a);
            const float rescale = expf(top - new_top);      // 0 the first time
            const float weight_a = expf(dot_a - new_top), weight_b = pair ? expf(dot_b - new_top) : 0.0f;
            denominator = denominator * rescale + weight_a + weight_b;
            top = new_top;
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                float x[n], y[n];
                unpack_row<T>(a[i], x);
                unpack_row<T>(b[i], y);
#pragma unroll
                for (int j = 0; j < n; ++j) sums[i][j] = fmaf(weight_b, y[j], fmaf(sums[i][j], rescale, weight_a * x[j]));
            }
        }
        key = stop;      // the step of two may have overshot by one
    }
    if (splits > 1) {
        float* record = partial + ((static_cast<size_t>(token) * heads + head) * splits + split) * (rank + 2);
        if (lane == 0) { record[0] = top; record[1] = denominator; }
#pragma unroll
        for (int i = 0; i < kPer; ++i)
#pragma unroll
            for (int j = 0; j < n; ++j) {
                const int column = (lane + 32 * i) * n + j;
                if (column < rank) record[2 + column] = sums[i][j];
            }
        return;
    }
    float rescale = 1.0f;
    if (sinks) {
        const float sink = sinks[head];
        const float new_top = fmaxf(top, sink);
        rescale = expf(top - new_top);
        denominator = denominator * rescale + expf(sink - new_top);
    }
    const float inverse = rescale / denominator;
#pragma unroll
    for (int i = 0; i < kPer; ++i)
#pragma unroll
        for (int j = 0; j < n; ++j) {
            const int column = (lane + 32 * i) * n + j;
            if (column < rank) out[(static_cast<size_t>(token) * heads + head) * rank + column] = from_float<T>(sums[i][j] * inverse);
        }
}

// One block per (token, head): joins the ranges of a context in their order.
template <typename T>
__global__ void latent_merge_kernel(const float* __restrict__ partial, const float* __restrict__ sinks, T* __restrict__ out, int heads, int rank, int splits) {
    grid_dependents_launch();
    grid_dependency_wait();
    const size_t item = blockIdx.x;
    const float* records = partial + item * splits * (rank + 2);
    float top = -INFINITY;
    for (int split = 0; split < splits; ++split) top = fmaxf(top, records[static_cast<size_t>(split) * (rank + 2)]);
    const float sink = sinks ? sinks[item % heads] : -INFINITY;
    const float all_top = fmaxf(top, sink);
    float denominator = sinks ? expf(sink - all_top) : 0.0f;
    for (int split = 0; split < splits; ++split) {
        const float* record = records + static_cast<size_t>(split) * (rank + 2);
        denominator += expf(record[0] - all_top) * record[1];
    }
    for (int column = threadIdx.x; column < rank; column += blockDim.x) {
        float sum = 0.0f;
        for (int split = 0; split < splits; ++split) {
            const float* record = records + static_cast<size_t>(split) * (rank + 2);
            sum = fmaf(expf(record[0] - all_top), record[2 + column], sum);
        }
        out[item * rank + column] = from_float<T>(sum / denominator);
    }
}

// For prompts that start at position 0: every head's full key [expanded unrotated part | rotated shared part] and value
// [expanded | zeros up to the key's width] go to pages of their own (sequence s owns pages s * pages_per_sequence ...), and
// every head's query [unrotated | rotated] to rows side by side, so that the attention kernels of ordinary heads serve them.
// `expanded` holds, per token, all heads' unrotated keys and then all heads' values.  One block per token.
template <typename T>
__global__ void __launch_bounds__(256)
latent_expand_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ down, long long down_stride, const T* __restrict__ expanded,
                     T* __restrict__ queries, T* __restrict__ key_pages, T* __restrict__ value_pages, const float* __restrict__ inv_freq, int rotary,
                     const int* __restrict__ positions, const int* __restrict__ token_seq, int pages_per_sequence, int page_tokens, int heads,
                     int head_dim, int rot, int rank, int value_dim) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int token = blockIdx.x, position = positions[token];
    const int width = head_dim + rot;
    const size_t page = static_cast<size_t>(token_seq[token]) * pages_per_sequence + position / page_tokens;
    const T* q_row = q + static_cast<size_t>(token) * q_stride;
    const T* shared_key = down + static_cast<size_t>(token) * down_stride + rank;
    const T* expanded_row = expanded + static_cast<size_t>(token) * heads * (head_dim + value_dim);
    for (int item = threadIdx.x; item < heads * width; item += blockDim.x) {
        const int head = item / width, column = item % width;
        float query, key;
        if (column < head_dim) {
            query = to_float(q_row[head * width + column]);
            key = to_float(expanded_row[head * head_dim + column]);
        } else {
            const int e = column - head_dim, first = e & ~1;
            const T* q_rot = q_row + head * width + head_dim;
            query = to_float(q_rot[e]);
            key = to_float(shared_key[e]);
            if (first + 1 < rotary) {
                float sine, cosine;
                sincosf(static_cast<float>(position) * inv_freq[first / 2], &sine, &cosine);
                const float qu = to_float(q_rot[first]), qw = to_float(q_rot[first + 1]);
                const float ku = to_float(shared_key[first]), kw = to_float(shared_key[first + 1]);
                query = (e & 1) ? qw * cosine + qu * sine : qu * cosine - qw * sine;
                key = (e & 1) ? kw * cosine + ku * sine : ku * cosine - kw * sine;
            }
        }
        queries[(static_cast<size_t>(token) * heads + head) * width + column] = from_float<T>(query);
        const size_t slot = ((page * heads + head) * page_tokens + position % page_tokens) * width + column;
        key_pages[slot] = from_float<T>(key);
        value_pages[slot] = column < value_dim ? expanded_row[heads * head_dim + head * value_dim + column] : from_float<T>(0.0f);
    }
}

// out[token, head, :value_dim] = values[token, head, :value_dim] * sigmoid(gate[token, head, :]) where a head's values are the
// first `value_dim` of `width` elements.
template <typename T>
__global__ void head_gate_kernel(const T* __restrict__ values, const T* __restrict__ gate, long long gate_stride, T* __restrict__ out, int heads,
                                 int width, int value_dim) {
    grid_dependents_launch();
    grid_dependency_wait();
    const size_t token = blockIdx.x;
    for (int item = threadIdx.x; item < heads * value_dim; item += blockDim.x) {
        const int head = item / value_dim, column = item % value_dim;
        float value = to_float(values[(token * heads + head) * width + column]);
        if (gate) value *= 1.0f / (1.0f + expf(-to_float(gate[token * gate_stride + item])));
        out[token * heads * value_dim + item] = from_float<T>(value);
    }
}

template <typename T>
int launch_vec(const void* queries, const void* rows, void* out, const float* sinks, const int* positions, const int* token_seq, const int* page_rows,
               int page_stride, int page_tokens, int tokens, int heads, int rank, int rot, float scale, int window, int splits, float* partial, cudaStream_t s) {
    const int warps = heads < kMaxWarps ? heads : kMaxWarps;
    tau_launch(latent_attention_vec_kernel<T>, dim3(tokens, (heads + kMaxWarps - 1) / kMaxWarps, splits), dim3(warps * 32), 0, s, static_cast<const T*>(queries),
               static_cast<const T*>(rows), static_cast<T*>(out), sinks, positions, token_seq, page_rows, page_stride, page_tokens, heads, rank, rot, scale,
               window, splits, partial);
    if (splits > 1) {
        const int status = tau_launch_status();
        if (status != 0) return status;
        tau_launch(latent_merge_kernel<T>, dim3(tokens * heads), dim3(128), 0, s, static_cast<const float*>(partial), sinks, static_cast<T*>(out), heads, rank, splits);
    }
    return tau_launch_status();
}

}  // namespace

// Floats of scratch that `splits` ranges need.
TAU_EXPORT long long tau_latent_attention_scratch(int tokens, int heads, int rank, int splits) {
    return splits > 1 ? static_cast<long long>(tokens) * heads * splits * (rank + 2) : 0;
}

TAU_EXPORT int tau_latent_prepare(int dtype, const void* down, long long down_stride, const float* latent_weight, float eps, const void* q,
                                  long long q_stride, void* queries, void* rows, const float* inv_freq, int rotary, const int* positions,
                                  const int* token_seq, const int* page_rows, int page_stride, int page_tokens, int tokens, int heads,
                                  int head_dim, int rot, int rank, int write_rows, void* latent_out, void* stream) {
    if (tokens <= 0) return 0;
    if (!q || !positions || !token_seq || heads <= 0 || rank <= 0 || rot < 0 || (rotary > 0 && !inv_freq) || rotary > rot
        || (write_rows && (!down || !latent_weight || !rows || !page_rows)))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TAU_F32)
        tau_launch(latent_prepare_kernel<float>, dim3(tokens), dim3(256), 0, s, static_cast<const float*>(down), down_stride, latent_weight, eps,
                   static_cast<const float*>(q), q_stride, static_cast<float*>(queries), static_cast<float*>(rows), inv_freq, rotary, positions,
                   token_seq, page_rows, page_stride, page_tokens, heads, head_dim, rot, rank, write_rows, static_cast<float*>(latent_out));
    else if (dtype == TAU_BF16)
        tau_launch(latent_prepare_kernel<bf16>, dim3(tokens), dim3(256), 0, s, static_cast<const bf16*>(down), down_stride, latent_weight, eps,
                   static_cast<const bf16*>(q), q_stride, static_cast<bf16*>(queries), static_cast<bf16*>(rows), inv_freq, rotary, positions,
                   token_seq, page_rows, page_stride, page_tokens, heads, head_dim, rot, rank, write_rows, static_cast<bf16*>(latent_out));
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}

TAU_EXPORT int tau_latent_attention(int dtype, const void* queries, const void* rows, void* out, const float* sinks, const int* positions,
                                    const int* token_seq, const int* page_rows, int page_stride, int page_tokens, int tokens, int heads, int rank,
                                    int rot, float scale, int window, int splits, float* partial, long long partial_floats, void* stream) {
    if (tokens <= 0) return 0;
    if (!queries || !rows || !out || !positions || !token_seq || !page_rows || heads <= 0 || rank <= 0 || rank > 32 * kMaxOwned || rot < 0 || splits < 1)
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Rows that are whole 16-byte vectors take the kernel that reads them as such; others the one that stages tiles.
    const int per_vector = dtype == TAU_BF16 ? 8 : 4;
    if ((rank + rot) % per_vector == 0 && rank + rot <= kVectorWidth && (dtype == TAU_BF16 || dtype == TAU_F32)) {
        if (splits > 1 && (!partial || partial_floats < tau_latent_attention_scratch(tokens, heads, rank, splits))) return cudaErrorInvalidValue;
        if (dtype == TAU_BF16)
            return launch_vec<bf16>(queries, rows, out, sinks, positions, token_seq, page_rows, page_stride, page_tokens, tokens, heads, rank, rot, scale, window, splits, partial, s);
        return launch_vec<float>(queries, rows, out, sinks, positions, token_seq, page_rows, page_stride, page_tokens, tokens, heads, rank, rot, scale, window, splits, partial, s);
    }
    const int warps = heads < kMaxWarps ? heads : kMaxWarps;
    const int width = rank + rot;
    const size_t bytes = (static_cast<size_t>(kTile) * (width + 1) + static_cast<size_t>(warps) * width) * sizeof(float);
    dim3 grid(tokens, (heads + kMaxWarps - 1) / kMaxWarps), block(warps * 32);
    cudaError_t status = cudaSuccess;
    if (dtype == TAU_F32) {
        if (bytes > 48 * 1024) status = cudaFuncSetAttribute(latent_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
        if (status != cudaSuccess) return status;
        tau_launch(latent_attention_kernel<float>, grid, block, bytes, s, static_cast<const float*>(queries), static_cast<const float*>(rows),
                   static_cast<float*>(out), sinks, positions, token_seq, page_rows, page_stride, page_tokens, heads, rank, rot, scale, window);
    } else if (dtype == TAU_BF16) {
        if (bytes > 48 * 1024) status = cudaFuncSetAttribute(latent_attention_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
        if (status != cudaSuccess) return status;
        tau_launch(latent_attention_kernel<bf16>, grid, block, bytes, s, static_cast<const bf16*>(queries), static_cast<const bf16*>(rows),
                   static_cast<bf16*>(out), sinks, positions, token_seq, page_rows, page_stride, page_tokens, heads, rank, rot, scale, window);
    } else {
        return cudaErrorInvalidValue;
    }
    return tau_launch_status();
}

TAU_EXPORT int tau_latent_expand(int dtype, const void* q, long long q_stride, const void* down, long long down_stride, const void* expanded, void* queries,
                                 void* key_pages, void* value_pages, const float* inv_freq, int rotary, const int* positions, const int* token_seq,
                                 int pages_per_sequence, int page_tokens, int tokens, int heads, int head_dim, int rot, int rank, int value_dim, void* stream) {
    if (tokens <= 0) return 0;
    if (!q || !down || !expanded || !queries || !key_pages || !value_pages || !positions || !token_seq || heads <= 0 || head_dim <= 0 || rot < 0
        || value_dim <= 0 || value_dim > head_dim + rot || rotary > rot || (rotary > 0 && !inv_freq) || pages_per_sequence <= 0)
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TAU_BF16)
        tau_launch(latent_expand_kernel<bf16>, dim3(tokens), dim3(256), 0, s, static_cast<const bf16*>(q), q_stride, static_cast<const bf16*>(down), down_stride,
                   static_cast<const bf16*>(expanded), static_cast<bf16*>(queries), static_cast<bf16*>(key_pages), static_cast<bf16*>(value_pages), inv_freq,
                   rotary, positions, token_seq, pages_per_sequence, page_tokens, heads, head_dim, rot, rank, value_dim);
    else if (dtype == TAU_F32)
        tau_launch(latent_expand_kernel<float>, dim3(tokens), dim3(256), 0, s, static_cast<const float*>(q), q_stride, static_cast<const float*>(down), down_stride,
                   static_cast<const float*>(expanded), static_cast<float*>(queries), static_cast<float*>(key_pages), static_cast<float*>(value_pages), inv_freq,
                   rotary, positions, token_seq, pages_per_sequence, page_tokens, heads, head_dim, rot, rank, value_dim);
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}

TAU_EXPORT int tau_head_gate(int dtype, const void* values, const void* gate, long long gate_stride, void* out, int tokens, int heads, int width,
                             int value_dim, void* stream) {
    if (tokens <= 0) return 0;
    if (!values || !out || heads <= 0 || value_dim <= 0 || value_dim > width) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TAU_BF16)
        tau_launch(head_gate_kernel<bf16>, dim3(tokens), dim3(256), 0, s, static_cast<const bf16*>(values), static_cast<const bf16*>(gate), gate_stride,
                   static_cast<bf16*>(out), heads, width, value_dim);
    else if (dtype == TAU_F32)
        tau_launch(head_gate_kernel<float>, dim3(tokens), dim3(256), 0, s, static_cast<const float*>(values), static_cast<const float*>(gate), gate_stride,
                   static_cast<float*>(out), heads, width, value_dim);
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}
