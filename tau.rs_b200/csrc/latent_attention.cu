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
constexpr int kMaxOwned = 16;      // latent columns per lane: rank <= 512

// One block per token.
template <typename T>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const T* __restrict__ down, long long down_stride, const float* __restrict__ latent_weight, float eps,
                      const T* __restrict__ q, long long q_stride, T* __restrict__ queries, T* __restrict__ rows,
                      const float* __restrict__ inv_freq, int rotary, const int* __restrict__ positions, const int* __restrict__ token_seq,
                      const int* __restrict__ page_rows, int page_stride, int page_tokens, int heads, int head_dim, int rot, int rank, int write_rows) {
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
        for (int column = threadIdx.x; column < rank; column += blockDim.x)
            target[column] = from_float<T>(to_float(source[column]) * inverse * latent_weight[column]);
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

}  // namespace

TAU_EXPORT int tau_latent_prepare(int dtype, const void* down, long long down_stride, const float* latent_weight, float eps, const void* q,
                                  long long q_stride, void* queries, void* rows, const float* inv_freq, int rotary, const int* positions,
                                  const int* token_seq, const int* page_rows, int page_stride, int page_tokens, int tokens, int heads,
                                  int head_dim, int rot, int rank, int write_rows, void* stream) {
    if (tokens <= 0) return 0;
    if (!q || !queries || !positions || !token_seq || heads <= 0 || rank <= 0 || rot < 0 || (rotary > 0 && !inv_freq) || rotary > rot
        || (write_rows && (!down || !latent_weight || !rows || !page_rows)))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TAU_F32)
        tau_launch(latent_prepare_kernel<float>, dim3(tokens), dim3(256), 0, s, static_cast<const float*>(down), down_stride, latent_weight, eps,
                   static_cast<const float*>(q), q_stride, static_cast<float*>(queries), static_cast<float*>(rows), inv_freq, rotary, positions,
                   token_seq, page_rows, page_stride, page_tokens, heads, head_dim, rot, rank, write_rows);
    else if (dtype == TAU_BF16)
        tau_launch(latent_prepare_kernel<bf16>, dim3(tokens), dim3(256), 0, s, static_cast<const bf16*>(down), down_stride, latent_weight, eps,
                   static_cast<const bf16*>(q), q_stride, static_cast<bf16*>(queries), static_cast<bf16*>(rows), inv_freq, rotary, positions,
                   token_seq, page_rows, page_stride, page_tokens, heads, head_dim, rot, rank, write_rows);
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}

TAU_EXPORT int tau_latent_attention(int dtype, const void* queries, const void* rows, void* out, const float* sinks, const int* positions,
                                    const int* token_seq, const int* page_rows, int page_stride, int page_tokens, int tokens, int heads, int rank,
                                    int rot, float scale, int window, void* stream) {
    if (tokens <= 0) return 0;
    if (!queries || !rows || !out || !positions || !token_seq || !page_rows || heads <= 0 || rank <= 0 || rank > 32 * kMaxOwned || rot < 0)
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
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
