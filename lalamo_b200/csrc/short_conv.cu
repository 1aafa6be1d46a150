// Gated short convolution over a ragged batch of request portions, with per-request state.
//
// proj[t] = [B (dim) ; C (dim) ; x (dim)]  (the in-projection's output, in this order)
// u[t]    = T(B[t] * x[t])
// hist    = [state (K-1 rows) ; u of this portion]
// c[j]    = sum_k w[ch, k] * hist[j + k]            (w[ch, K-1] multiplies the current token)
// y[t]    = T(C[t] * T(c + bias))
// new state = hist[q_len : q_len + K-1]             (keeps the tail of the old state when q_len < K-1)
#include "common.cuh"

namespace lb {

constexpr int kConvTokensPerBlock = 8;

template <typename T>
__device__ __forceinline__ float gated_input(const T* proj, size_t token, int dim, int channel) {
    const T* row = proj + token * 3 * static_cast<size_t>(dim);
    return round_to<T>(to_float(row[channel]) * to_float(row[2 * static_cast<size_t>(dim) + channel]));
}

template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ proj, const T* __restrict__ state, const float* __restrict__ weight,
                                  const float* __restrict__ bias, T* __restrict__ out,
                                  const int* __restrict__ token_segment, const int* __restrict__ segment_start,
                                  const int* __restrict__ segment_slot, int tokens, int dim, int kernel_size,
                                  int num_slots, int* status) {
    const int channel = blockIdx.y * blockDim.x + threadIdx.x;
    if (channel >= dim) return;
    const int history = kernel_size - 1;
    const float* w = weight + static_cast<size_t>(channel) * kernel_size;
    const float b = bias ? bias[channel] : 0.0f;
    const int first = blockIdx.x * kConvTokensPerBlock;
    const int last = min(tokens, first + kConvTokensPerBlock);
    for (int token = first; token < last; ++token) {
        const int segment = token_segment[token];
        const int j = token - segment_start[segment];   // index within the portion
        const int slot = segment_slot[segment];
        if (slot < 0 || slot >= num_slots) {
            report_error(status, kBadSlot);
            continue;
        }
        const T* slot_state = state + static_cast<size_t>(slot) * history * dim;
        float sum = 0.0f;
        for (int k = 0; k < kernel_size; ++k) {
            const int index = j + k - history;   // index into u of this portion; negative -> state
            float value;
            if (index >= 0) {
                value = gated_input(proj, static_cast<size_t>(token - j + index), dim, channel);
            } else {
                value = to_float(slot_state[static_cast<size_t>(history + index) * dim + channel]);
            }
            sum += w[k] * value;
        }
        const float conv = round_to<T>(sum + b);
        const float gate = to_float(proj[static_cast<size_t>(token) * 3 * dim + dim + channel]);
        out[static_cast<size_t>(token) * dim + channel] = from_float<T>(gate * conv);
    }
}

// The same for bfloat16 with dim % 8 == 0, 16-byte accesses.  One token's 8 channels:
// TAPS > 0 fixes the number of taps at compile time, so that the loads of all taps leave together.
template <int TAPS>
__device__ __forceinline__ void short_conv_one_token(const __nv_bfloat16* __restrict__ proj, const __nv_bfloat16* __restrict__ state,
                                                     const float* __restrict__ weight, const float* __restrict__ bias, __nv_bfloat16* __restrict__ out,
                                                     const int* __restrict__ token_segment, const int* __restrict__ segment_start,
                                                     const int* __restrict__ segment_slot, int token, int channel, int dim, int kernel_size, int num_slots,
                                                     int* status) {
    if (TAPS > 0) kernel_size = TAPS;
    const int history = kernel_size - 1;
    const int segment = token_segment[token];
    const int start = segment_start[segment];
    const int j = token - start;
    const int slot = segment_slot[segment];
    if (slot < 0 || slot >= num_slots) {
        report_error(status, kBadSlot);
        return;
    }
    float sum[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) sum[c] = bias ? bias[channel + c] : 0.0f;
    // The taps of this thread's 8 channels are 8 * TAPS consecutive floats, 16-byte aligned.
    float taps[TAPS > 0 ? 8 * TAPS : 1];
    if (TAPS > 0) {
        const float4* source = reinterpret_cast<const float4*>(weight + static_cast<size_t>(channel) * TAPS);
#pragma unroll
        for (int i = 0; i < 2 * TAPS; ++i) {
            const float4 four = source[i];
            taps[4 * i] = four.x;
            taps[4 * i + 1] = four.y;
            taps[4 * i + 2] = four.z;
            taps[4 * i + 3] = four.w;
        }
    }
    float conv[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) conv[c] = 0.0f;
#pragma unroll
    for (int k = 0; k < (TAPS > 0 ? TAPS : kernel_size); ++k) {
        const int i = j + k - history;
        float value[8];
        if (i >= 0) {
            const __nv_bfloat16* row = proj + static_cast<size_t>(start + i) * 3 * dim;
            const uint4 gate_raw = *reinterpret_cast<const uint4*>(row + channel);
            const uint4 x_raw = *reinterpret_cast<const uint4*>(row + 2 * static_cast<size_t>(dim) + channel);
            const __nv_bfloat162* gate = reinterpret_cast<const __nv_bfloat162*>(&gate_raw);
            const __nv_bfloat162* x = reinterpret_cast<const __nv_bfloat162*>(&x_raw);
#pragma unroll
            for (int pair = 0; pair < 4; ++pair) {
                const float2 a = __bfloat1622float2(gate[pair]), b = __bfloat1622float2(x[pair]);
                value[2 * pair] = round_to<__nv_bfloat16>(a.x * b.x);
                value[2 * pair + 1] = round_to<__nv_bfloat16>(a.y * b.y);
            }
        } else {
            const uint4 raw = *reinterpret_cast<const uint4*>(state + (static_cast<size_t>(slot) * history + history + i) * dim + channel);
            const __nv_bfloat162* held = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int pair = 0; pair < 4; ++pair) {
                const float2 a = __bfloat1622float2(held[pair]);
                value[2 * pair] = a.x;
                value[2 * pair + 1] = a.y;
            }
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) conv[c] += (TAPS > 0 ? taps[c * (TAPS > 0 ? TAPS : 1) + k] : weight[static_cast<size_t>(channel + c) * kernel_size + k]) * value[c];
    }
    const uint4 post_raw = *reinterpret_cast<const uint4*>(proj + static_cast<size_t>(token) * 3 * dim + dim + channel);
    const __nv_bfloat162* post = reinterpret_cast<const __nv_bfloat162*>(&post_raw);
    uint4 result_raw;
    __nv_bfloat162* result = reinterpret_cast<__nv_bfloat162*>(&result_raw);
#pragma unroll
    for (int pair = 0; pair < 4; ++pair) {
        const float2 gate = __bfloat1622float2(post[pair]);
        result[pair] = __floats2bfloat162_rn(gate.x * round_to<__nv_bfloat16>(conv[2 * pair] + sum[2 * pair]),
                                             gate.y * round_to<__nv_bfloat16>(conv[2 * pair + 1] + sum[2 * pair + 1]));
    }
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(token) * dim + channel) = result_raw;
}

// One thread per (token, 8 channels): steps of few tokens, and numbers of taps without a kernel of their own.
template <int TAPS>
__global__ void short_conv_bf16x8_kernel(const __nv_bfloat16* __restrict__ proj, const __nv_bfloat16* __restrict__ state,
                                         const float* __restrict__ weight, const float* __restrict__ bias, __nv_bfloat16* __restrict__ out,
                                         const int* __restrict__ token_segment, const int* __restrict__ segment_start,
                                         const int* __restrict__ segment_slot, int tokens, int dim, int kernel_size, int num_slots,
                                         int* status) {
    // Launched to start early: resident when the in-projection ends; the state update after it may take its place in turn.
    wait_for_previous_kernel();
    allow_next_kernel();
    const int groups = dim / 8;
    const size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= static_cast<size_t>(tokens) * groups) return;
    const int token = static_cast<int>(index / groups);
    const int channel = static_cast<int>(index - static_cast<size_t>(token) * groups) * 8;
    short_conv_one_token<TAPS>(proj, state, weight, bias, out, token_segment, segment_start, segment_slot, token, channel, dim, kernel_size, num_slots, status);
}

// Steps of many tokens: one thread per (kConvRun consecutive tokens, 8 channels).  Where its tokens belong to one
// portion, the thread loads every row of the in-projection once (the gated inputs of a token serve the TAPS tokens
// after it), all loads leaving together; a run that crosses a portion's end goes token by token.
constexpr int kConvRun = 4;
constexpr int kConvRunMinTokens = 256;   // below, a thread per token fills the GPU better

__device__ __forceinline__ void gated_inputs_bf16x8(float (&value)[8], const __nv_bfloat16* __restrict__ row, int dim, int channel) {
    const uint4 gate_raw = *reinterpret_cast<const uint4*>(row + channel);
    const uint4 x_raw = *reinterpret_cast<const uint4*>(row + 2 * static_cast<size_t>(dim) + channel);
    const __nv_bfloat162* gate = reinterpret_cast<const __nv_bfloat162*>(&gate_raw);
    const __nv_bfloat162* x = reinterpret_cast<const __nv_bfloat162*>(&x_raw);
#pragma unroll
    for (int pair = 0; pair < 4; ++pair) {
        const float2 a = __bfloat1622float2(gate[pair]), b = __bfloat1622float2(x[pair]);
        value[2 * pair] = round_to<__nv_bfloat16>(a.x * b.x);
        value[2 * pair + 1] = round_to<__nv_bfloat16>(a.y * b.y);
    }
}

template <int TAPS>
__global__ void short_conv_bf16x8_run_kernel(const __nv_bfloat16* __restrict__ proj, const __nv_bfloat16* __restrict__ state,
                                             const float* __restrict__ weight, const float* __restrict__ bias, __nv_bfloat16* __restrict__ out,
                                             const int* __restrict__ token_segment, const int* __restrict__ segment_start,
                                             const int* __restrict__ segment_slot, int tokens, int dim, int num_slots, int* status) {
    wait_for_previous_kernel();   // launched to start early, as the kernel above
    allow_next_kernel();
    constexpr int history = TAPS - 1;
    const int groups = dim / 8;
    const int runs = (tokens + kConvRun - 1) / kConvRun;
    const size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= static_cast<size_t>(runs) * groups) return;
    const int run = static_cast<int>(index / groups);
    const int channel = static_cast<int>(index - static_cast<size_t>(run) * groups) * 8;
    const int first = run * kConvRun, last = min(tokens, first + kConvRun) - 1;
    // The run's own rows depend on nothing but its place in the batch: they are asked for before the lists say
    // which portion the run belongs to.
    uint4 gate_raw[kConvRun], x_raw[kConvRun], post_raw[kConvRun];
#pragma unroll
    for (int t = 0; t < kConvRun; ++t) {
        const __nv_bfloat16* row = proj + static_cast<size_t>(min(first + t, last)) * 3 * dim;
        gate_raw[t] = *reinterpret_cast<const uint4*>(row + channel);
        post_raw[t] = *reinterpret_cast<const uint4*>(row + dim + channel);
        x_raw[t] = *reinterpret_cast<const uint4*>(row + 2 * static_cast<size_t>(dim) + channel);
    }
    float taps[8 * TAPS];
    {
        const float4* source = reinterpret_cast<const float4*>(weight + static_cast<size_t>(channel) * TAPS);
#pragma unroll
        for (int i = 0; i < 2 * TAPS; ++i) {
            const float4 four = source[i];
            taps[4 * i] = four.x;
            taps[4 * i + 1] = four.y;
            taps[4 * i + 2] = four.z;
            taps[4 * i + 3] = four.w;
        }
    }
    const int segment = token_segment[first];
    if (last - first + 1 < kConvRun || token_segment[last] != segment) {
        for (int token = first; token <= last; ++token)
            short_conv_one_token<TAPS>(proj, state, weight, bias, out, token_segment, segment_start, segment_slot, token, channel, dim, TAPS, num_slots, status);
        return;
    }
    const int start = segment_start[segment];
    const int slot = segment_slot[segment];
    if (slot < 0 || slot >= num_slots) {
        report_error(status, kBadSlot);
        return;
    }
    const int j = first - start;   // the first token's index within its portion
    // u[r]: the gated input history + kConvRun rows back from the run's last token, oldest first
    float u[history + kConvRun][8];
#pragma unroll
    for (int r = 0; r < history; ++r) {
        const int i = j - history + r;
        if (i >= 0) {
            gated_inputs_bf16x8(u[r], proj + static_cast<size_t>(start + i) * 3 * dim, dim, channel);
        } else {
            const uint4 raw = *reinterpret_cast<const uint4*>(state + (static_cast<size_t>(slot) * history + history + i) * dim + channel);
            const __nv_bfloat162* held = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int pair = 0; pair < 4; ++pair) {
                const float2 a = __bfloat1622float2(held[pair]);
                u[r][2 * pair] = a.x;
                u[r][2 * pair + 1] = a.y;
            }
        }
    }
#pragma unroll
    for (int t = 0; t < kConvRun; ++t) {
        const __nv_bfloat162* gate = reinterpret_cast<const __nv_bfloat162*>(&gate_raw[t]);
        const __nv_bfloat162* x = reinterpret_cast<const __nv_bfloat162*>(&x_raw[t]);
#pragma unroll
        for (int pair = 0; pair < 4; ++pair) {
            const float2 a = __bfloat1622float2(gate[pair]), b = __bfloat1622float2(x[pair]);
            u[history + t][2 * pair] = round_to<__nv_bfloat16>(a.x * b.x);
            u[history + t][2 * pair + 1] = round_to<__nv_bfloat16>(a.y * b.y);
        }
    }
    float sum[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) sum[c] = bias ? bias[channel + c] : 0.0f;
#pragma unroll
    for (int t = 0; t < kConvRun; ++t) {
        float conv[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) conv[c] = 0.0f;
#pragma unroll
        for (int k = 0; k < TAPS; ++k) {
#pragma unroll
            for (int c = 0; c < 8; ++c) conv[c] += taps[c * TAPS + k] * u[t + k][c];
        }
        const __nv_bfloat162* post = reinterpret_cast<const __nv_bfloat162*>(&post_raw[t]);
        uint4 result_raw;
        __nv_bfloat162* result = reinterpret_cast<__nv_bfloat162*>(&result_raw);
#pragma unroll
        for (int pair = 0; pair < 4; ++pair) {
            const float2 gate = __bfloat1622float2(post[pair]);
            result[pair] = __floats2bfloat162_rn(gate.x * round_to<__nv_bfloat16>(conv[2 * pair] + sum[2 * pair]),
                                                 gate.y * round_to<__nv_bfloat16>(conv[2 * pair + 1] + sum[2 * pair + 1]));
        }
        *reinterpret_cast<uint4*>(out + static_cast<size_t>(first + t) * dim + channel) = result_raw;
    }
}

// A step in which every portion is one token (decoding): one thread per (token, 8 channels) does all of it, the state
// update included (nobody else touches its request's state), in one kernel instead of three.  The in-projection may
// come as the partial sums of its K slices (`partials[slice][token][3 dim]`, float32, `slice_stride` floats apart), which
// the thread adds in slice order and rounds to bfloat16 as the product's own epilogue would have; else `proj` holds it.
__global__ void short_conv_single_kernel(const float* __restrict__ partials, int slices, size_t slice_stride, const __nv_bfloat16* __restrict__ proj,
                                         __nv_bfloat16* __restrict__ state, const float* __restrict__ weight, const float* __restrict__ bias,
                                         __nv_bfloat16* __restrict__ out, const int* __restrict__ token_segment, const int* __restrict__ segment_slot,
                                         int tokens, int dim, int kernel_size, int num_slots, int* status) {
    wait_for_previous_kernel();   // launched to start early
    allow_next_kernel();
    const int groups = dim / 8;
    const size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= static_cast<size_t>(tokens) * groups) return;
    const int token = static_cast<int>(index / groups);
    const int channel = static_cast<int>(index - static_cast<size_t>(token) * groups) * 8;
    const int history = kernel_size - 1;
    const int slot = segment_slot[token_segment[token]];
    if (slot < 0 || slot >= num_slots) {
        report_error(status, kBadSlot);
        return;
    }
    // B (multiplies x), C (multiplies the convolution) and x of this token's channels
    float part[3][8];
    if (slices > 0) {
        const float* row = partials + static_cast<size_t>(token) * 3 * dim + channel;
#pragma unroll
        for (int which = 0; which < 3; ++which) {
            float total[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
            for (int s = 0; s < slices; ++s) {
                const float4 low = *reinterpret_cast<const float4*>(row + s * slice_stride + static_cast<size_t>(which) * dim);
                const float4 high = *reinterpret_cast<const float4*>(row + s * slice_stride + static_cast<size_t>(which) * dim + 4);
                total[0] += low.x, total[1] += low.y, total[2] += low.z, total[3] += low.w;
                total[4] += high.x, total[5] += high.y, total[6] += high.z, total[7] += high.w;
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) part[which][c] = round_to<__nv_bfloat16>(total[c]);
        }
    } else {
        const __nv_bfloat16* row = proj + static_cast<size_t>(token) * 3 * dim + channel;
#pragma unroll
        for (int which = 0; which < 3; ++which) {
            const uint4 raw = *reinterpret_cast<const uint4*>(row + static_cast<size_t>(which) * dim);
            const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int pair = 0; pair < 4; ++pair) {
                const float2 two = __bfloat1622float2(pairs[pair]);
                part[which][2 * pair] = two.x;
                part[which][2 * pair + 1] = two.y;
            }
        }
    }
    float u[8], conv[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        u[c] = round_to<__nv_bfloat16>(part[0][c] * part[2][c]);
        conv[c] = 0.0f;
    }
    // the taps over the held rows, oldest first, each row handed one place down as it is read; then the token's own
    __nv_bfloat16* held = state + static_cast<size_t>(slot) * history * dim + channel;
    for (int k = 0; k < history; ++k) {
        const uint4 raw = *reinterpret_cast<const uint4*>(held + static_cast<size_t>(k) * dim);
        const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int pair = 0; pair < 4; ++pair) {
            const float2 two = __bfloat1622float2(pairs[pair]);
            conv[2 * pair] += weight[static_cast<size_t>(channel + 2 * pair) * kernel_size + k] * two.x;
            conv[2 * pair + 1] += weight[static_cast<size_t>(channel + 2 * pair + 1) * kernel_size + k] * two.y;
        }
        if (k > 0) *reinterpret_cast<uint4*>(held + static_cast<size_t>(k - 1) * dim) = raw;
    }
    uint4 newest_raw, result_raw;
    __nv_bfloat162* newest = reinterpret_cast<__nv_bfloat162*>(&newest_raw);
    __nv_bfloat162* result = reinterpret_cast<__nv_bfloat162*>(&result_raw);
#pragma unroll
    for (int c = 0; c < 8; ++c) conv[c] += weight[static_cast<size_t>(channel + c) * kernel_size + history] * u[c];
#pragma unroll
    for (int pair = 0; pair < 4; ++pair) {
        newest[pair] = __floats2bfloat162_rn(u[2 * pair], u[2 * pair + 1]);
        const float b0 = bias ? bias[channel + 2 * pair] : 0.0f, b1 = bias ? bias[channel + 2 * pair + 1] : 0.0f;
        result[pair] = __floats2bfloat162_rn(part[1][2 * pair] * round_to<__nv_bfloat16>(conv[2 * pair] + b0),
                                             part[1][2 * pair + 1] * round_to<__nv_bfloat16>(conv[2 * pair + 1] + b1));
    }
    if (history > 0) *reinterpret_cast<uint4*>(held + static_cast<size_t>(history - 1) * dim) = newest_raw;
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(token) * dim + channel) = result_raw;
}

// grid (segments, ceil(dim / threads)).  Runs after short_conv_kernel on the same stream.
template <typename T>
__global__ void short_conv_state_kernel(const T* __restrict__ proj, T* __restrict__ state,
                                        const int* __restrict__ segment_start, const int* __restrict__ segment_length,
                                        const int* __restrict__ segment_slot, int dim, int kernel_size, int num_slots) {
    // Launched to start early: the convolution before it has read the old state when this wait returns, and the
    // product after this kernel may ask for its weights meanwhile.
    wait_for_previous_kernel();
    allow_next_kernel();
    const int segment = blockIdx.x;
    const int channel = blockIdx.y * blockDim.x + threadIdx.x;
    if (channel >= dim) return;
    const int history = kernel_size - 1;
    const int slot = segment_slot[segment];
    if (slot < 0 || slot >= num_slots) return;
    const int start = segment_start[segment], length = segment_length[segment];
    T* slot_state = state + static_cast<size_t>(slot) * history * dim;
    // Row r of the new state is hist[length + r]; hist index >= r + 1, so rows are read before
    // they are overwritten when r ascends.
    for (int r = 0; r < history; ++r) {
        const int index = length + r;
        T value;
        if (index < history) {
            value = slot_state[static_cast<size_t>(index) * dim + channel];
        } else {
            value = from_float<T>(gated_input(proj, static_cast<size_t>(start + index - history), dim, channel));
        }
        slot_state[static_cast<size_t>(r) * dim + channel] = value;
    }
}

}  // namespace lb

extern "C" {

int lb_short_conv(const void* proj, void* state, const float* weight, const float* bias, void* out,
                  const int* token_segment, const int* segment_start, const int* segment_length,
                  const int* segment_slot, int tokens, int segments, int dim, int kernel_size, int num_slots, int dtype,
                  int* status, cudaStream_t stream) {
    if (tokens == 0 || segments == 0) return 0;
    if (kernel_size < 1) return -2;
    const int threads = 128;
    const dim3 grid((tokens + lb::kConvTokensPerBlock - 1) / lb::kConvTokensPerBlock, (dim + threads - 1) / threads);
    const dim3 state_grid(segments, (dim + threads - 1) / threads);
    if (dtype == lb::kBFloat16 && dim % 8 == 0) {
        const size_t work = static_cast<size_t>(tokens) * (dim / 8);
        auto kernel = kernel_size == 2   ? lb::short_conv_bf16x8_kernel<2>
                      : kernel_size == 3 ? lb::short_conv_bf16x8_kernel<3>
                      : kernel_size == 4 ? lb::short_conv_bf16x8_kernel<4>
                                         : lb::short_conv_bf16x8_kernel<0>;
        if (tokens >= lb::kConvRunMinTokens && kernel_size >= 2 && kernel_size <= 4) {
            auto run_kernel = kernel_size == 2 ? lb::short_conv_bf16x8_run_kernel<2> : kernel_size == 3 ? lb::short_conv_bf16x8_run_kernel<3> : lb::short_conv_bf16x8_run_kernel<4>;
            const size_t run_work = static_cast<size_t>((tokens + lb::kConvRun - 1) / lb::kConvRun) * (dim / 8);
            lb::launch_overlapped(run_kernel, dim3(static_cast<unsigned>((run_work + 127) / 128)), dim3(128), 0, stream,
                static_cast<const __nv_bfloat16*>(proj), static_cast<const __nv_bfloat16*>(state), weight, bias, static_cast<__nv_bfloat16*>(out),
                token_segment, segment_start, segment_slot, tokens, dim, num_slots, status);
        } else {
            lb::launch_overlapped(kernel, dim3(static_cast<unsigned>((work + 255) / 256)), dim3(256), 0, stream,
                static_cast<const __nv_bfloat16*>(proj), static_cast<const __nv_bfloat16*>(state), weight, bias, static_cast<__nv_bfloat16*>(out),
                token_segment, segment_start, segment_slot, tokens, dim, kernel_size, num_slots, status);
        }
        if (kernel_size > 1) {
            lb::launch_overlapped(lb::short_conv_state_kernel<__nv_bfloat16>, state_grid, dim3(threads), 0, stream,
                static_cast<const __nv_bfloat16*>(proj), static_cast<__nv_bfloat16*>(state), segment_start, segment_length, segment_slot, dim, kernel_size,
                num_slots);
        }
        return LB_LAUNCH_RESULT();
    }
    LB_DISPATCH_DTYPE(dtype, {
        lb::short_conv_kernel<T><<<grid, threads, 0, stream>>>(static_cast<const T*>(proj), static_cast<const T*>(state), weight,
                                                               bias, static_cast<T*>(out), token_segment, segment_start,
                                                               segment_slot, tokens, dim, kernel_size, num_slots, status);
        if (kernel_size > 1) {
            lb::short_conv_state_kernel<T><<<state_grid, threads, 0, stream>>>(static_cast<const T*>(proj), static_cast<T*>(state),
                                                                               segment_start, segment_length, segment_slot, dim,
                                                                               kernel_size, num_slots);
        }
    })
    return LB_LAUNCH_RESULT();
}

// The same for a step of single tokens (every portion one token), in one kernel.  Either `partials` ([slices, tokens, 3 dim]
// float32 partial sums of the in-projection, slices > 0) or `proj` ([tokens, 3 dim] bfloat16, slices == 0).  dim % 8 == 0.
int lb_short_conv_single(const float* partials, int slices, const void* proj, void* state, const float* weight, const float* bias, void* out,
                         const int* token_segment, const int* segment_slot, int tokens, int dim, int kernel_size, int num_slots, int* status,
                         cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (kernel_size < 1 || dim < 8 || dim % 8 != 0 || slices < 0 || (slices > 0 ? partials == nullptr : proj == nullptr)) return -2;
    if ((reinterpret_cast<uintptr_t>(partials) | reinterpret_cast<uintptr_t>(proj) | reinterpret_cast<uintptr_t>(state) | reinterpret_cast<uintptr_t>(out)) & 15) return -2;
    const size_t work = static_cast<size_t>(tokens) * (dim / 8);
    return static_cast<int>(lb::launch_overlapped(lb::short_conv_single_kernel, dim3(static_cast<unsigned>((work + 127) / 128)), dim3(128), 0, stream, partials, slices,
                                                  static_cast<size_t>(tokens) * 3 * dim, static_cast<const __nv_bfloat16*>(proj), static_cast<__nv_bfloat16*>(state), weight,
                                                  bias, static_cast<__nv_bfloat16*>(out), token_segment, segment_slot, tokens, dim, kernel_size, num_slots, status));
}

}  // extern "C"
