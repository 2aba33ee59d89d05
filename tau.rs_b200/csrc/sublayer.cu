// Kernels of a block arrangement that normalises what a sublayer returns instead of what it reads, on a residual stream kept
// in 32-bit:
//
//   causal taps     read[t] = x[t] + sum_j w[j, :] * x[t - taps + 1 + j], a short causal convolution over time on each channel whose
//                   rows before a run's first token come from the sequence's state (its last taps - 1 inputs; zeros at the start)
//   taps state      the state after the run: the last taps - 1 inputs of the sequence
//   gated add norm  target = source + norm(branch * sigmoid(gate)) * weight + bias, the norm centred (layer norm) or not (RMS)
//   side gate       g[t, c] = gelu_tanh(z[t, c]) * table[token[t], offset + c]
//   unit add mix    X = x + y / rms(y) * weight; kept as the run's result; out = sum_j mix[j] * results[j]
//   norm rows       out[i] = norm(values[rows[i]]) * weight + bias
//   activation      relu(z)^2
//
// Statistics, sums and the stream are 32-bit; what products read next is rounded once to the activations' dtype.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float load_as_float(const void* base, int code, size_t index) {
    return code == TAU_BF16 ? __bfloat162float(static_cast<const bf16*>(base)[index]) : static_cast<const float*>(base)[index];
}

__device__ __forceinline__ float sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// V consecutive elements at once (V = 1, or 4 where every row starts on a 16-byte boundary and the width is a multiple of 4).
template <int V> struct Pack { float v[V]; };

template <int V>
__device__ __forceinline__ Pack<V> load_pack(const void* base, int code, size_t index) {
    Pack<V> pack;
    if constexpr (V == 4) {
        if (code == TAU_BF16) {
            const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const bf16*>(base) + index);
            pack.v[0] = __uint_as_float(raw.x << 16);
            pack.v[1] = __uint_as_float(raw.x & 0xffff0000u);
            pack.v[2] = __uint_as_float(raw.y << 16);
            pack.v[3] = __uint_as_float(raw.y & 0xffff0000u);
        } else {
            const float4 raw = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + index);
            pack.v[0] = raw.x; pack.v[1] = raw.y; pack.v[2] = raw.z; pack.v[3] = raw.w;
        }
    } else {
        pack.v[0] = load_as_float(base, code, index);
    }
    return pack;
}

template <int V>
__device__ __forceinline__ void store_pack(float* base, size_t index, const Pack<V>& pack) {
    if constexpr (V == 4) *reinterpret_cast<float4*>(base + index) = make_float4(pack.v[0], pack.v[1], pack.v[2], pack.v[3]);
    else base[index] = pack.v[0];
}

template <int V>
__device__ __forceinline__ void store_pack(bf16* base, size_t index, const Pack<V>& pack) {
    if constexpr (V == 4) {
        const __nv_bfloat162 low = __floats2bfloat162_rn(pack.v[0], pack.v[1]), high = __floats2bfloat162_rn(pack.v[2], pack.v[3]);
        uint2 raw;
        raw.x = *reinterpret_cast<const unsigned*>(&low);
        raw.y = *reinterpret_cast<const unsigned*>(&high);
        *reinterpret_cast<uint2*>(base + index) = raw;
    } else {
        base[index] = __float2bfloat16_rn(pack.v[0]);
    }
}

// grid: tokens.  state [slots, taps - 1, width]; row `taps - 1 + s` of it stands for the sequence's input at run-local index s < 0.
// `shift_state`: every sequence brings one token, so the block of a token is the only reader of its sequence's state and moves it
// on itself (each thread the channels it has just read): rows go down by one and the token becomes the last.
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
causal_taps_kernel(const float* __restrict__ x, const float* __restrict__ weight, float* state, const int* __restrict__ token_seq,
                   const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, T* __restrict__ read_out, T* __restrict__ plain_out,
                   int width, int taps, int shift_state) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int token = blockIdx.x, seq = token_seq[token], first = cu_seqlens[seq], local = token - first;
    float* kept = state + static_cast<size_t>(seq_slot[seq]) * (taps - 1) * width;
    for (int column = threadIdx.x * V; column < width; column += blockDim.x * V) {
        const Pack<V> own = load_pack<V>(x, TAU_F32, static_cast<size_t>(token) * width + column);
        Pack<V> sum;
#pragma unroll
        for (int e = 0; e < V; ++e) sum.v[e] = 0.0f;
        for (int j = 0; j < taps; ++j) {
            const int source = local - (taps - 1) + j;
            const Pack<V> value = source >= 0 ? load_pack<V>(x, TAU_F32, static_cast<size_t>(first + source) * width + column)
                                              : load_pack<V>(kept, TAU_F32, static_cast<size_t>(taps - 1 + source) * width + column);
            const Pack<V> tap = load_pack<V>(weight, TAU_F32, static_cast<size_t>(j) * width + column);      // weight [taps, width]
#pragma unroll
            for (int e = 0; e < V; ++e) sum.v[e] = fmaf(tap.v[e], value.v[e], sum.v[e]);
        }
#pragma unroll
        for (int e = 0; e < V; ++e) sum.v[e] += own.v[e];
        store_pack<V>(read_out, static_cast<size_t>(token) * width + column, sum);
        if (plain_out) store_pack<V>(plain_out, static_cast<size_t>(token) * width + column, own);
        if (shift_state) {
            for (int i = 0; i + 2 < taps; ++i)
                store_pack<V>(kept, static_cast<size_t>(i) * width + column, load_pack<V>(kept, TAU_F32, static_cast<size_t>(i + 1) * width + column));
            store_pack<V>(kept, static_cast<size_t>(taps - 2) * width + column, own);
        }
    }
}

// grid: (sequences, ceil(width / threads)).  Runs after every reader of the old state in stream order.  A thread owns a channel and walks the rows upwards:
// row i takes the input at run-local index count - (taps - 1) + i, which for a negative index is the old row i + count, not yet overwritten.
__global__ void __launch_bounds__(kThreads)
taps_state_kernel(const float* __restrict__ x, float* __restrict__ state, const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                  int width, int taps) {
    grid_dependents_launch();
    grid_dependency_wait();
    const int seq = blockIdx.x, first = cu_seqlens[seq], count = cu_seqlens[seq + 1] - first;
    float* kept = state + static_cast<size_t>(seq_slot[seq]) * (taps - 1) * width;
    const int column = blockIdx.y * blockDim.x + threadIdx.x;
    if (column < width) {
        for (int i = 0; i < taps - 1; ++i) {
            const int source = count - (taps - 1) + i;
            kept[static_cast<size_t>(i) * width + column] = source >= 0 ? x[static_cast<size_t>(first + source) * width + column]
                                                                         : kept[static_cast<size_t>(taps - 1 + source) * width + column];
        }
    }
}

// grid: rows.  `target` may be `source`.  Dynamic shared memory: width floats.
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
gated_add_norm_kernel(const float* source, float* target, const void* __restrict__ branch, int branch_code,
                      const void* __restrict__ gate, int gate_code, long long gate_stride, const float* __restrict__ weight,
                      const float* __restrict__ bias, T* __restrict__ copy_out, int width, float eps, int centred) {
    grid_dependents_launch();
    grid_dependency_wait();
    extern __shared__ __align__(16) float gated[];
    __shared__ float scratch[33];
    const size_t base = static_cast<size_t>(blockIdx.x) * width;
    float total = 0.0f;
    for (int column = threadIdx.x * V; column < width; column += blockDim.x * V) {
        Pack<V> value = load_pack<V>(branch, branch_code, base + column);
        if (gate) {
            const Pack<V> z = load_pack<V>(gate, gate_code, static_cast<size_t>(blockIdx.x) * gate_stride + column);
#pragma unroll
            for (int e = 0; e < V; ++e) value.v[e] *= sigmoid(z.v[e]);
        }
        store_pack<V>(gated, column, value);
#pragma unroll
        for (int e = 0; e < V; ++e) total += value.v[e];
    }
    const float mean = centred ? block_sum(total, scratch) / static_cast<float>(width) : 0.0f;
    float squares = 0.0f;
    for (int column = threadIdx.x * V; column < width; column += blockDim.x * V) {
        const Pack<V> value = load_pack<V>(gated, TAU_F32, column);       // each thread reads back what it wrote itself
#pragma unroll
        for (int e = 0; e < V; ++e) squares += (value.v[e] - mean) * (value.v[e] - mean);
    }
    const float inverse = 1.0f / sqrtf(block_sum(squares, scratch) / static_cast<float>(width) + eps);
    for (int column = threadIdx.x * V; column < width; column += blockDim.x * V) {
        Pack<V> value = load_pack<V>(gated, TAU_F32, column);
        const Pack<V> scale = load_pack<V>(weight, TAU_F32, column), before = load_pack<V>(source, TAU_F32, base + column);
#pragma unroll
        for (int e = 0; e < V; ++e) value.v[e] = (value.v[e] - mean) * inverse * scale.v[e];
        if (bias) {
            const Pack<V> shift = load_pack<V>(bias, TAU_F32, column);
#pragma unroll
            for (int e = 0; e < V; ++e) value.v[e] += shift.v[e];
        }
#pragma unroll
        for (int e = 0; e < V; ++e) value.v[e] += before.v[e];
        store_pack<V>(target, base + column, value);
        if (copy_out) store_pack<V>(copy_out, base + column, value);
    }
}

__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
side_gate_kernel(const T* z, const T* __restrict__ table, const int* __restrict__ tokens, T* out, long long count,
                 int dim, int table_width, int offset, int vocab) {
    grid_dependents_launch();
    grid_dependency_wait();
    const long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= count) return;
    const int row = static_cast<int>(index / dim), column = static_cast<int>(index % dim);
    const int token = tokens[row];
    const float entry = token >= 0 && token < vocab ? to_float(table[static_cast<size_t>(token) * table_width + offset + column]) : 0.0f;
    out[index] = from_float<T>(gelu_tanh(to_float(z[index])) * entry);
}

// grid: rows.  X = source + y / rms(y) * weight (X = source where there is no y) goes to `result` (the slot of this run among `results`, or the stream itself);
// with `mix` (count floats, count - 1 earlier results [count - 1][rows][width] starting at `results`) `out` = sum_j mix[j] * results[j],
// the newest result being X.  Dynamic shared memory: width floats.
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
unit_add_mix_kernel(const float* source, const void* __restrict__ y, int y_code, const float* __restrict__ weight, float* result,
                    const float* __restrict__ results, long long result_stride, const float* __restrict__ mix, int count, float* __restrict__ out,
                    T* __restrict__ copy_out, int width, float eps) {
    grid_dependents_launch();
    grid_dependency_wait();
    extern __shared__ __align__(16) float held[];
    __shared__ float scratch[33];
    const size_t base = static_cast<size_t>(blockIdx.x) * width;
    float inverse = 0.0f;
    if (y) {
        float squares = 0.0f;
        for (int column = threadIdx.x * V; column < width; column += blockDim.x * V) {
            const Pack<V> value = load_pack<V>(y, y_code, base + column);
            store_pack<V>(held, column, value);
#pragma unroll
            for (int e = 0; e < V; ++e) squares += value.v[e] * value.v[e];
        }
        inverse = 1.0f / sqrtf(block_sum(squares, scratch) / static_cast<float>(width) + eps);
    }
    for (int column = threadIdx.x * V; column < width; column += blockDim.x * V) {
        Pack<V> newest = load_pack<V>(source, TAU_F32, base + column);
        if (y) {
            const Pack<V> value = load_pack<V>(held, TAU_F32, column), scale = load_pack<V>(weight, TAU_F32, column);
#pragma unroll
            for (int e = 0; e < V; ++e) newest.v[e] += value.v[e] * inverse * scale.v[e];
        }
        store_pack<V>(result, base + column, newest);
        Pack<V> value = newest;
        if (mix) {
#pragma unroll
            for (int e = 0; e < V; ++e) value.v[e] = 0.0f;
            for (int j = 0; j + 1 < count; ++j) {
                const Pack<V> earlier = load_pack<V>(results, TAU_F32, static_cast<size_t>(j) * result_stride + base + column);
                const float share = mix[j];
#pragma unroll
                for (int e = 0; e < V; ++e) value.v[e] = fmaf(share, earlier.v[e], value.v[e]);
            }
            const float share = mix[count - 1];
#pragma unroll
            for (int e = 0; e < V; ++e) value.v[e] = fmaf(share, newest.v[e], value.v[e]);
            store_pack<V>(out, base + column, value);
        }
        if (copy_out) store_pack<V>(copy_out, base + column, value);
    }
}

// grid: output rows.  Layer norm (centred) or RMS norm of values[rows[i]] (32-bit or T), weight and optional bias.
template <typename T>
__global__ void __launch_bounds__(kThreads)
norm_rows_kernel(const void* __restrict__ values, int values_code, const int* __restrict__ rows, const float* __restrict__ weight,
                 const float* __restrict__ bias, T* __restrict__ out, int width, float eps, int centred) {
    grid_dependents_launch();
    grid_dependency_wait();
    extern __shared__ float held[];
    __shared__ float scratch[33];
    const size_t base = static_cast<size_t>(rows ? rows[blockIdx.x] : blockIdx.x) * width;
    float total = 0.0f;
    for (int column = threadIdx.x; column < width; column += blockDim.x) {
        const float value = load_as_float(values, values_code, base + column);
        held[column] = value;
        total += value;
    }
    const float mean = centred ? block_sum(total, scratch) / static_cast<float>(width) : 0.0f;
    float squares = 0.0f;
    for (int column = threadIdx.x; column < width; column += blockDim.x) {
        const float deviation = held[column] - mean;
        squares += deviation * deviation;
    }
    const float inverse = 1.0f / sqrtf(block_sum(squares, scratch) / static_cast<float>(width) + eps);
    for (int column = threadIdx.x; column < width; column += blockDim.x) {
        float value = (held[column] - mean) * inverse * weight[column];
        if (bias) value += bias[column];
        out[static_cast<size_t>(blockIdx.x) * width + column] = from_float<T>(value);
    }
}

// A thread takes 16 bytes (V elements) where the tensors allow it.
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
relu_squared_kernel(const T* z, T* out, long long count) {
    grid_dependents_launch();
    grid_dependency_wait();
    const long long index = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * V;
    if (index >= count) return;
    if constexpr (V == 1) {
        const float value = fmaxf(to_float(z[index]), 0.0f);
        out[index] = from_float<T>(value * value);
    } else {
        uint4 raw = *reinterpret_cast<const uint4*>(z + index);
        T* values = reinterpret_cast<T*>(&raw);
#pragma unroll
        for (int e = 0; e < V; ++e) {
            const float value = fmaxf(to_float(values[e]), 0.0f);
            values[e] = from_float<T>(value * value);
        }
        *reinterpret_cast<uint4*>(out + index) = raw;
    }
}

// Whether every pointer given (null ones aside) lies on a 16-byte boundary.
template <typename... Pointers>
bool aligned16(Pointers... pointers) {
    return (((reinterpret_cast<uintptr_t>(pointers)) | ...) & 15) == 0;
}

template <typename Kernel>
int allow_shared(Kernel kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return 0;
    return static_cast<int>(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
}

}  // namespace

TAU_EXPORT int tau_causal_taps(int dtype, const float* x, const float* weight, float* state, const int* token_seq, const int* cu_seqlens,
                               const int* seq_slot, void* read_out, void* plain_out, int tokens, int sequences, int width, int taps, int update,
                               int all_single, void* stream) {
    if (tokens <= 0) return 0;
    if (!x || (!weight && taps > 0) || (!state && taps > 1) || !token_seq || !cu_seqlens || !seq_slot || !read_out || sequences <= 0 || width <= 0 || taps < 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int shift = (update && taps > 1 && all_single && tokens == sequences) ? 1 : 0;
    const bool wide = width % 4 == 0 && aligned16(x, weight, state, read_out, plain_out);
    if (dtype == TAU_F32) {
        auto kernel = wide ? causal_taps_kernel<float, 4> : causal_taps_kernel<float, 1>;
        tau_launch(kernel, dim3(tokens), dim3(kThreads), 0, s, x, weight, state, token_seq, cu_seqlens, seq_slot,
                   static_cast<float*>(read_out), static_cast<float*>(plain_out), width, taps, shift);
    } else if (dtype == TAU_BF16) {
        auto kernel = wide ? causal_taps_kernel<bf16, 4> : causal_taps_kernel<bf16, 1>;
        tau_launch(kernel, dim3(tokens), dim3(kThreads), 0, s, x, weight, state, token_seq, cu_seqlens, seq_slot,
                   static_cast<bf16*>(read_out), static_cast<bf16*>(plain_out), width, taps, shift);
    } else {
        return cudaErrorInvalidValue;
    }
    int status = tau_launch_status();
    if (status != 0 || !update || taps < 2 || shift) return status;
    tau_launch(taps_state_kernel, dim3(sequences, (width + kThreads - 1) / kThreads), dim3(kThreads), 0, s, x, state, cu_seqlens, seq_slot, width, taps);
    return tau_launch_status();
}

TAU_EXPORT int tau_gated_add_norm(int dtype, const float* source, float* target, const void* branch, int branch_dtype, const void* gate, int gate_dtype,
                                  long long gate_stride, const float* weight, const float* bias, void* copy_out, int rows, int width, float eps,
                                  int centred, void* stream) {
    if (rows <= 0) return 0;
    if (!source || !target || !branch || !weight || width <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t bytes = static_cast<size_t>(width) * sizeof(float);
    const bool wide = width % 4 == 0 && gate_stride % 8 == 0 && aligned16(source, target, branch, gate, weight, bias, copy_out);
    if (dtype == TAU_F32) {
        auto kernel = wide ? gated_add_norm_kernel<float, 4> : gated_add_norm_kernel<float, 1>;
        if (int status = allow_shared(kernel, bytes)) return status;
        tau_launch(kernel, dim3(rows), dim3(kThreads), bytes, s, source, target, branch, branch_dtype, gate, gate_dtype, gate_stride,
                   weight, bias, static_cast<float*>(copy_out), width, eps, centred);
    } else if (dtype == TAU_BF16) {
        auto kernel = wide ? gated_add_norm_kernel<bf16, 4> : gated_add_norm_kernel<bf16, 1>;
        if (int status = allow_shared(kernel, bytes)) return status;
        tau_launch(kernel, dim3(rows), dim3(kThreads), bytes, s, source, target, branch, branch_dtype, gate, gate_dtype, gate_stride,
                   weight, bias, static_cast<bf16*>(copy_out), width, eps, centred);
    } else {
        return cudaErrorInvalidValue;
    }
    return tau_launch_status();
}

TAU_EXPORT int tau_side_gate(int dtype, const void* z, const void* table, const int* tokens, void* out, int rows, int dim, int table_width, int offset,
                             int vocab, void* stream) {
    if (rows <= 0) return 0;
    if (!z || !table || !tokens || !out || dim <= 0 || offset < 0 || offset + dim > table_width || vocab <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long long count = static_cast<long long>(rows) * dim;
    const dim3 grid(static_cast<unsigned>((count + kThreads - 1) / kThreads));
    if (dtype == TAU_F32)
        tau_launch(side_gate_kernel<float>, grid, dim3(kThreads), 0, s, static_cast<const float*>(z), static_cast<const float*>(table), tokens,
                   static_cast<float*>(out), count, dim, table_width, offset, vocab);
    else if (dtype == TAU_BF16)
        tau_launch(side_gate_kernel<bf16>, grid, dim3(kThreads), 0, s, static_cast<const bf16*>(z), static_cast<const bf16*>(table), tokens,
                   static_cast<bf16*>(out), count, dim, table_width, offset, vocab);
    else
        return cudaErrorInvalidValue;
    return tau_launch_status();
}

TAU_EXPORT int tau_unit_add_mix(int dtype, const float* source, const void* y, int y_dtype, const float* weight, float* result, const float* results,
                                long long result_stride, const float* mix, int count, float* out, void* copy_out, int rows, int width, float eps,
                                void* stream) {
    if (rows <= 0) return 0;
    if (!source || (y && !weight) || !result || width <= 0 || (mix && (count < 1 || !out || (count > 1 && !results)))) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t bytes = static_cast<size_t>(width) * sizeof(float);
    const bool wide = width % 4 == 0 && result_stride % 4 == 0 && aligned16(source, y, weight, result, results, out, copy_out);
    if (dtype == TAU_F32) {
        auto kernel = wide ? unit_add_mix_kernel<float, 4> : unit_add_mix_kernel<float, 1>;
        if (int status = allow_shared(kernel, bytes)) return status;
        tau_launch(kernel, dim3(rows), dim3(kThreads), bytes, s, source, y, y_dtype, weight, result, results, result_stride, mix, count, out,
                   static_cast<float*>(copy_out), width, eps);
    } else if (dtype == TAU_BF16) {
        auto kernel = wide ? unit_add_mix_kernel<bf16, 4> : unit_add_mix_kernel<bf16, 1>;
        if (int status = allow_shared(kernel, bytes)) return status;
        tau_launch(kernel, dim3(rows), dim3(kThreads), bytes, s, source, y, y_dtype, weight, result, results, result_stride, mix, count, out,
                   static_cast<bf16*>(copy_out), width, eps);
    } else {
        return cudaErrorInvalidValue;
    }
    return tau_launch_status();
}

TAU_EXPORT int tau_norm_rows(int dtype, const void* values, int values_dtype, const int* rows, const float* weight, const float* bias, void* out,
                             int out_rows, int width, float eps, int centred, void* stream) {
    if (out_rows <= 0) return 0;
    if (!values || !weight || !out || width <= 0) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t bytes = static_cast<size_t>(width) * sizeof(float);
    if (dtype == TAU_F32) {
        if (int status = allow_shared(norm_rows_kernel<float>, bytes)) return status;
        tau_launch(norm_rows_kernel<float>, dim3(out_rows), dim3(kThreads), bytes, s, values, values_dtype, rows, weight, bias, static_cast<float*>(out), width, eps, centred);
    } else if (dtype == TAU_BF16) {
        if (int status = allow_shared(norm_rows_kernel<bf16>, bytes)) return status;
        tau_launch(norm_rows_kernel<bf16>, dim3(out_rows), dim3(kThreads), bytes, s, values, values_dtype, rows, weight, bias, static_cast<bf16*>(out), width, eps, centred);
    } else {
        return cudaErrorInvalidValue;
    }
    return tau_launch_status();
}

TAU_EXPORT int tau_relu_squared(int dtype, const void* z, void* out, long long count, void* stream) {
    if (count <= 0) return 0;
    if (!z || !out) return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool wide = count % 8 == 0 && aligned16(z, out);
    const int per_thread = !wide ? 1 : dtype == TAU_BF16 ? 8 : 4;
    const dim3 grid(static_cast<unsigned>((count / per_thread + kThreads - 1) / kThreads));
    if (dtype == TAU_F32) tau_launch(wide ? relu_squared_kernel<float, 4> : relu_squared_kernel<float, 1>, grid, dim3(kThreads), 0, s, static_cast<const float*>(z), static_cast<float*>(out), count);
    else if (dtype == TAU_BF16) tau_launch(wide ? relu_squared_kernel<bf16, 8> : relu_squared_kernel<bf16, 1>, grid, dim3(kThreads), 0, s, static_cast<const bf16*>(z), static_cast<bf16*>(out), count);
    else return cudaErrorInvalidValue;
    return tau_launch_status();
}
