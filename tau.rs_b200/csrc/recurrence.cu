// Linear recurrences with a matrix state per head, for runs of new tokens and for single tokens alike:
//
//     S_t = a_t S_(t-1) + b_t k_t v_t^T          o_t = S_t^T q_t            (S is key_dim x value_dim)
//
// Two gatings.  Decay: a_t is a constant of the head, b_t = 1 (linear attention with a decay per head).
// Exponential: a log input gate i_t and a log forget gate f_t per head and token, both from soft-capped
// pre-activations (i = cap tanh(x / cap), f = logsigmoid(cap tanh(y / cap))), a running maximum
// m_t = max(f_t + m_(t-1), i_t) that starts at 0, a_t = exp(f_t + m_(t-1) - m_t), b_t = exp(i_t - m_t), a normaliser
// n_t = a_t n_(t-1) + b_t k_t, and o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6).
//
// The state is 32-bit and lives in the cache, one record per (slot, head): value_dim (+1) columns of key_dim
// numbers each, the extra column being n (which obeys the recurrence of a value that is always 1), then m.
// One block owns a (sequence, head, tile of columns) and walks the sequence's new tokens in order; a thread keeps
// its share of one column in registers, so a token costs one pass over key_dim per thread and two barriers.
// Everything is computed in 32-bit; q, k, v arrive in the activations' dtype.  TAU_KEY_DIM fixes key_dim.
#include "common.cuh"

#ifndef TAU_KEY_DIM
#error "compile with -DTAU_KEY_DIM=<key elements per head>"
#endif

namespace {

constexpr int kDim = TAU_KEY_DIM;
constexpr int kSplit = kDim <= 16 ? 1 : kDim <= 32 ? 2 : kDim <= 64 ? 4 : kDim <= 128 ? 8 : kDim <= 256 ? 16 : 32;   // threads that share a column
constexpr int kRows = (kDim + kSplit - 1) / kSplit;                               // key rows per thread
// Columns of a block (n included): 32, or 16 where 32 would leave SMs without a block.

__device__ __forceinline__ float activate(float value, int activation) { return activation ? value / (1.0f + expf(-value)) : value; }

// The gates' pre-activations become log gates in place, for all tokens at once: what does not depend on the token before
// is not computed inside the walk.  gates [tokens, 2 heads]: inputs first, then forgets.
__global__ void log_gates_kernel(float* __restrict__ gates, long long count, int heads, float gate_cap) {
    grid_dependents_launch();
    grid_dependency_wait();
    for (long long index = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; index < count; index += static_cast<long long>(gridDim.x) * blockDim.x) {
        const float capped = gate_cap * tanhf(gates[index] / gate_cap);
        const bool forget = (index / heads) & 1;
        gates[index] = forget ? fminf(capped, 0.0f) - log1pf(expf(-fabsf(capped))) : capped;     // logsigmoid for the forget gate
    }
}

template <typename T, int kColumns>
__global__ void __launch_bounds__(kColumns * kSplit)
linear_recurrence_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long long stride,
                         const float* __restrict__ gates, const float* __restrict__ decays, float* __restrict__ state, long long slot_stride,
                         const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, float* __restrict__ out,
                         int heads, int value_dim, int exponential, float gate_cap, float query_scale, int activation) {
    grid_dependents_launch();
    grid_dependency_wait();
    __shared__ float qs[2][kDim], ks[2][kDim], partial[2][kSplit][kColumns];
    const int head = blockIdx.x, sequence = blockIdx.y;
    const int columns = value_dim + (exponential ? 1 : 0);           // n rides as one more column of the state
    // A block serves a tile of value columns; with the exponential gating its last thread column serves n as well, in every
    // block (each needs n . q), and the first block alone writes n and m back.
    const int tile = exponential ? kColumns - 1 : kColumns;
    const int local = threadIdx.x % kColumns;
    const bool is_n = exponential && local == kColumns - 1;
    const int column = is_n ? value_dim : blockIdx.z * tile + local;
    const int part = threadIdx.x / kColumns, row0 = part * kRows;
    const bool live = is_n || column < value_dim;
    float* record = state + static_cast<size_t>(seq_slot[sequence]) * slot_stride + static_cast<size_t>(head) * (static_cast<size_t>(columns) * kDim + (exponential ? 1 : 0));
    float S[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) S[r] = (live && row0 + r < kDim) ? record[static_cast<size_t>(column) * kDim + row0 + r] : 0.0f;
    float m = exponential ? record[static_cast<size_t>(columns) * kDim] : 0.0f;
    const float decay = exponential ? 1.0f : decays[head];
    const int begin = cu_seqlens[sequence], end = cu_seqlens[sequence + 1];
    // Operands are asked for four tokens ahead, in four sets of registers that take turns: a token's q and k go into the free
    // half of qs/ks one token before they are used, its v and gates stay in their set until its turn, and the set is filled
    // again for the token four further on.  The walk then waits for memory at its start only.
    constexpr int kStage = (kDim + kColumns * kSplit - 1) / (kColumns * kSplit);
    constexpr int kAhead = 4;
    float next_q[kAhead][kStage], next_k[kAhead][kStage], next_v[kAhead], next_in[kAhead], next_forget[kAhead];
    auto fetch = [&](int set, int token) {
        if (token >= end) return;
        const size_t row = static_cast<size_t>(token) * stride;
#pragma unroll
        for (int i = 0; i < kStage; ++i) {
            const int d = threadIdx.x + i * kColumns * kSplit;
            if (d < kDim) {
                next_q[set][i] = to_float(q[row + head * kDim + d]);
                next_k[set][i] = to_float(k[row + head * kDim + d]);
            }
        }
        if (live && !is_n) next_v[set] = to_float(v[row + head * value_dim + column]);
        if (exponential) {
            next_in[set] = gates[static_cast<size_t>(token) * 2 * heads + head];
            next_forget[set] = gates[static_cast<size_t>(token) * 2 * heads + heads + head];
        }
    };
    auto publish = [&](int set, int half) {
#pragma unroll
        for (int i = 0; i < kStage; ++i) {
            const int d = threadIdx.x + i * kColumns * kSplit;
            if (d < kDim) {
                qs[half][d] = activate(next_q[set][i], activation) * query_scale;
                ks[half][d] = activate(next_k[set][i], activation);
            }
        }
    };
#pragma unroll
    for (int set = 0; set < kAhead; ++set) {
        next_v[set] = next_in[set] = next_forget[set] = 0.0f;
        fetch(set, begin + set);
    }
    if (begin < end) publish(0, 0);
    __syncthreads();
    for (int base = begin; base < end; base += kAhead) {
#pragma unroll
      for (int set = 0; set < kAhead; ++set) {
        const int token = base + set;
        if (token >= end) break;
        const int half = set & 1;                  // kAhead is even: the halves take turns with the tokens
        const float raw_value = next_v[set], raw_in = next_in[set], raw_forget = next_forget[set];
        float keep = decay, take = 1.0f;
        if (exponential) {
            const float log_in = raw_in, log_forget = raw_forget;     // made log gates by `log_gates_kernel`
            const float m_new = fmaxf(log_forget + m, log_in);
            keep = expf(log_forget + m - m_new);
            take = expf(log_in - m_new);
            m = m_new;
        }
        const float value = is_n ? 1.0f : live ? activate(raw_value, activation) : 0.0f;
        const float scaled = take * value;
        float sums[4] = {0.0f, 0.0f, 0.0f, 0.0f};      // four chains, so that a sum does not wait for the one before it
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            if (row0 + r < kDim) {
                S[r] = fmaf(keep, S[r], ks[half][row0 + r] * scaled);
                sums[r & 3] = fmaf(S[r], qs[half][row0 + r], sums[r & 3]);
            }
        }
        // One barrier per token: partial sums and the next token's q and k go to the halves of shared memory that nobody reads
        // now; behind the barrier the first thread of each column adds the parts up, and n's as well for the denominator.
        partial[half][part][local] = (sums[0] + sums[1]) + (sums[2] + sums[3]);
        if (token + 1 < end) publish((set + 1) % kAhead, half ^ 1);
        fetch(set, token + kAhead);                 // this set's q and k were published a token ago, its v and gates just used
        __syncthreads();
        if (part == 0 && live && !is_n) {
            float sum = 0.0f;
#pragma unroll
            for (int p = 0; p < kSplit; ++p) sum += partial[half][p][local];
            if (exponential) {
                float normaliser = 0.0f;
#pragma unroll
                for (int p = 0; p < kSplit; ++p) normaliser += partial[half][p][kColumns - 1];
                sum /= fmaxf(fabsf(normaliser), expf(-m)) + 1e-6f;
            }
            out[static_cast<size_t>(token) * heads * value_dim + head * value_dim + column] = sum;
        }
      }
    }
    if (live && (!is_n || blockIdx.z == 0)) {
#pragma unroll
        for (int r = 0; r < kRows; ++r)
            if (row0 + r < kDim) record[static_cast<size_t>(column) * kDim + row0 + r] = S[r];
    }
    if (exponential && blockIdx.z == 0 && threadIdx.x == 0) record[static_cast<size_t>(columns) * kDim] = m;
}

}  // namespace

TAU_EXPORT int tau_recurrence_key_dim() { return kDim; }

// q, k, v: rows `stride` elements apart, heads side by side.  gates [tokens, 2 heads] (exponential; pre-activations, turned into log
// gates in place) or decays [heads].
// state: records `slot_stride` floats apart per slot.  out [tokens, heads * value_dim], 32-bit.
TAU_EXPORT int tau_linear_recurrence(int dtype, const void* q, const void* k, const void* v, long long stride, float* gates,
                                     const float* decays, float* state, long long slot_stride, const int* cu_seqlens, const int* seq_slot,
                                     float* out, int tokens, int n_seqs, int heads, int value_dim, int exponential, float gate_cap, float query_scale,
                                     int activation, void* stream) {
    if (n_seqs <= 0) return 0;
    if (!q || !k || !v || !state || !cu_seqlens || !seq_slot || !out || heads <= 0 || value_dim <= 0 || (exponential ? !gates : !decays))
        return cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (exponential) {
        if (tokens <= 0) return cudaErrorInvalidValue;
        const long long count = static_cast<long long>(tokens) * 2 * heads;
        tau_launch(log_gates_kernel, dim3(static_cast<unsigned>((count + 255) / 256 < 1184 ? (count + 255) / 256 : 1184)), dim3(256), 0, s, gates, count, heads, gate_cap);
        const int status = tau_launch_status();
        if (status != 0) return status;
    }
    const int wide = exponential ? 31 : 32;
    const bool narrow = heads * n_seqs * ((value_dim + wide - 1) / wide) < 148 && kSplit <= 16;     // blocks of 16 columns reach more SMs
    const int tile = narrow ? (exponential ? 15 : 16) : wide;
    dim3 grid(heads, n_seqs, (value_dim + tile - 1) / tile), block((narrow ? 16 : 32) * kSplit);
    if (dtype != TAU_F32 && dtype != TAU_BF16) return cudaErrorInvalidValue;
#define TAU_RECURRENCE(T, COLUMNS)                                                                                                          \
    tau_launch(linear_recurrence_kernel<T, COLUMNS>, grid, block, 0, s, static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), \
               stride, gates, decays, state, slot_stride, cu_seqlens, seq_slot, out, heads, value_dim, exponential, gate_cap, query_scale, activation)
    if (dtype == TAU_F32) {
        if (narrow) TAU_RECURRENCE(float, 16); else TAU_RECURRENCE(float, 32);
    } else {
        if (narrow) TAU_RECURRENCE(bf16, 16); else TAU_RECURRENCE(bf16, 32);
    }
#undef TAU_RECURRENCE
    return tau_launch_status();
}
