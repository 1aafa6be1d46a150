// Per-head q/k norm + rotary embedding + paged K/V write, and the plain paged attention.
//
// The plain attention kernel is the 32-bit path's attention and the reference against which
// the tensor-core kernels are tested: one block per (token, head), keys visited in chunks that
// start at the first visible key, so the result does not depend on how a prompt was cut into
// steps or on what else is in the batch.
#include "common.cuh"

namespace lb {

struct PagedLayout {
    int page_size;
    int num_pages;
    int max_blocks;   // columns of the block table
    int num_groups;   // K/V heads
    int head_dim;
};

// Keys are stored [page][row][group][head_dim]; values transposed, [page][group][head_dim][row], so
// that the keys of one page are contiguous for each channel (the operand layout the tensor-core
// kernels want for the product of probabilities and values).

// Address of the key row of `position` of the request in `segment`, or nullptr if the block
// table has no valid page there.
template <typename T>
__device__ __forceinline__ T* page_row(T* pages, const int* block_table, const PagedLayout& layout, int segment,
                                       int position, int group) {
    const int block = position / layout.page_size;
    if (block >= layout.max_blocks) return nullptr;
    const int page = block_table[static_cast<size_t>(segment) * layout.max_blocks + block];
    if (page < 0 || page >= layout.num_pages) return nullptr;
    const size_t row = static_cast<size_t>(page) * layout.page_size + (position - block * layout.page_size);
    return pages + (row * layout.num_groups + group) * layout.head_dim;
}

// Address of channel 0 of the value of `position`; channel d lies `d * page_size` elements further.
template <typename T>
__device__ __forceinline__ T* value_column(T* pages, const int* block_table, const PagedLayout& layout, int segment,
                                           int position, int group) {
    const int block = position / layout.page_size;
    if (block >= layout.max_blocks) return nullptr;
    const int page = block_table[static_cast<size_t>(segment) * layout.max_blocks + block];
    if (page < 0 || page >= layout.num_pages) return nullptr;
    const size_t base = (static_cast<size_t>(page) * layout.num_groups + group) * layout.head_dim * layout.page_size;
    return pages + base + (position - block * layout.page_size);
}

// grid (tokens, num_heads + num_groups), one warp per head vector.
//   y < num_heads: query head -> q_out[token, head, :]
//   else: key head g -> K page row (norm + rope), and value head g copied to the V page row.
// Norm: T(x * rsqrt(mean x^2 + eps)) * T(w), rounded to T; rope in 32-bit on the rounded value:
//   out[d] = y[d] cos(a) + rot[d] sin(a), rot = concat(-y[half:], y[:half]), a = pos * inv_freq[d mod half].
template <typename T>
__global__ void qk_norm_rope_write_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_pages,
                                          T* __restrict__ v_pages, const float* __restrict__ q_weight,
                                          const float* __restrict__ k_weight, float eps, float scale_offset,
                                          const float* __restrict__ inv_freq, int rotary_dim,
                                          const int* __restrict__ positions, const int* __restrict__ token_segment,
                                          const int* __restrict__ block_table, PagedLayout layout, int num_heads,
                                          int write_kv, int* status) {
    // Launched to start early; once the kernel before it (the q/k/v product) is done, the attention after it
    // may start in turn and read the keys and values that this kernel does not write.
    wait_for_previous_kernel();
    allow_next_kernel();
    const int token = blockIdx.x;
    const int unit = blockIdx.y;
    const int lane = threadIdx.x;
    const int hd = layout.head_dim;
    const int width = (num_heads + 2 * layout.num_groups) * hd;
    const bool is_query = unit < num_heads;
    if (!is_query && !write_kv) return;
    const int group = unit - num_heads;
    const T* src = qkv + static_cast<size_t>(token) * width + static_cast<size_t>(unit) * hd;
    const float* weight = is_query ? q_weight : k_weight;
    const int position = positions[token];

    T* dst;
    if (is_query) {
        dst = q_out + (static_cast<size_t>(token) * num_heads + unit) * hd;
    } else {
        const int segment = token_segment[token];
        dst = page_row(k_pages, block_table, layout, segment, position, group);
        T* v_dst = value_column(v_pages, block_table, layout, segment, position, group);
        if (dst == nullptr || v_dst == nullptr) {
            if (lane == 0) report_error(status, kBadPage);
            return;
        }
        const T* v_src = qkv + static_cast<size_t>(token) * width + static_cast<size_t>(num_heads + layout.num_groups + group) * hd;
        for (int d = lane; d < hd; d += 32) v_dst[static_cast<size_t>(d) * layout.page_size] = v_src[d];
    }

    float inv = 1.0f;
    if (weight != nullptr) {
        float sum = 0.0f;
        for (int d = lane; d < hd; d += 32) {
            const float v = to_float(src[d]);
            sum += v * v;
        }
        sum = warp_sum(sum);
        inv = rsqrtf(sum / static_cast<float>(hd) + eps);
    }
    const int half = rotary_dim / 2;
    for (int d = lane; d < hd; d += 32) {
        float y = to_float(src[d]);
        if (weight != nullptr) y = round_to<T>(round_to<T>(y * inv) * round_to<T>(weight[d] + scale_offset));
        if (d < rotary_dim) {
            const int partner = d < half ? d + half : d - half;
            float other = to_float(src[partner]);
            if (weight != nullptr) other = round_to<T>(round_to<T>(other * inv) * round_to<T>(weight[partner] + scale_offset));
            const float angle = static_cast<float>(position) * inv_freq[d < half ? d : d - half];
            float sine, cosine;
            sincosf(angle, &sine, &cosine);
            const float rotated = d < half ? -other : other;
            y = y * cosine + rotated * sine;
        }
        dst[d] = from_float<T>(y);
    }
}

// The same work with a few blocks per token: the sines and cosines of the token's position are
// computed once per block, in shared memory, and serve its eight query or key heads (one warp per
// head, heads taken in turn).
constexpr int kTokenKernelUnits = 8;   // query or key heads per block of the per-token kernel

template <typename T>
__global__ void qk_norm_rope_write_token_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_pages,
                                                T* __restrict__ v_pages, const float* __restrict__ q_weight,
                                                const float* __restrict__ k_weight, float eps, float scale_offset,
                                                const float* __restrict__ inv_freq, int rotary_dim,
                                                const int* __restrict__ positions, const int* __restrict__ token_segment,
                                                const int* __restrict__ block_table, PagedLayout layout, int num_heads,
                                                int write_kv, int* status) {
    extern __shared__ float rotation[];   // cos[half], sin[half]
    const int token = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int hd = layout.head_dim;
    const int half = rotary_dim / 2;
    const int width = (num_heads + 2 * layout.num_groups) * hd;
    const int position = positions[token];
    const int segment = token_segment[token];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sine, cosine;
        sincosf(static_cast<float>(position) * inv_freq[i], &sine, &cosine);
        rotation[i] = cosine;
        rotation[half + i] = sine;
    }
    __syncthreads();
    const int units = num_heads + (write_kv ? layout.num_groups : 0);
    // grid.y shares out the heads: blocks of one token take kTokenKernelUnits of them each.
    const int unit_end = min(units, (static_cast<int>(blockIdx.y) + 1) * kTokenKernelUnits);
    for (int unit = blockIdx.y * kTokenKernelUnits + warp; unit < unit_end; unit += warps) {
        const bool is_query = unit < num_heads;
        const int group = unit - num_heads;
        const T* src = qkv + static_cast<size_t>(token) * width + static_cast<size_t>(unit) * hd;
        const float* weight = is_query ? q_weight : k_weight;
        T* dst;
        if (is_query) {
            dst = q_out + (static_cast<size_t>(token) * num_heads + unit) * hd;
        } else {
            dst = page_row(k_pages, block_table, layout, segment, position, group);
            T* v_dst = value_column(v_pages, block_table, layout, segment, position, group);
            if (dst == nullptr || v_dst == nullptr) {
                if (lane == 0) report_error(status, kBadPage);
                continue;
            }
            const T* v_src = qkv + static_cast<size_t>(token) * width + static_cast<size_t>(num_heads + layout.num_groups + group) * hd;
            for (int d = lane; d < hd; d += 32) v_dst[static_cast<size_t>(d) * layout.page_size] = v_src[d];
        }
        float inv = 1.0f;
        if (weight != nullptr) {
            float sum = 0.0f;
            for (int d = lane; d < hd; d += 32) {
                const float v = to_float(src[d]);
                sum += v * v;
            }
            sum = warp_sum(sum);
            inv = rsqrtf(sum / static_cast<float>(hd) + eps);
        }
        for (int d = lane; d < hd; d += 32) {
            float y = to_float(src[d]);
            if (weight != nullptr) y = round_to<T>(round_to<T>(y * inv) * round_to<T>(weight[d] + scale_offset));
            if (d < rotary_dim) {
                const int partner = d < half ? d + half : d - half;
                float other = to_float(src[partner]);
                if (weight != nullptr) other = round_to<T>(round_to<T>(other * inv) * round_to<T>(weight[partner] + scale_offset));
                const int i = d < half ? d : d - half;
                const float rotated = d < half ? -other : other;
                y = y * rotation[i] + rotated * rotation[half + i];
            }
            dst[d] = from_float<T>(y);
        }
    }
}

// The same work for bfloat16 and head sizes 16, 32, 64 and 128 with rotary_dim a multiple of 16: one
// block per token, one thread per 8 consecutive channels of a head (16-byte loads and stores), so that
// the 2, 4, 8 or 16 threads of a head are neighbours in a warp: the sum of squares is reduced and the
// rotation partner's normalised values are fetched by shuffles.  Sines and cosines of the token's
// position are computed once per block.
__global__ void qk_norm_rope_write_vector_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                                                 __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                                                 const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
                                                 float scale_offset, const float* __restrict__ inv_freq, int rotary_dim,
                                                 const int* __restrict__ positions, const int* __restrict__ token_segment,
                                                 const int* __restrict__ block_table, PagedLayout layout, int num_heads, int write_kv,
                                                 int* status) {
    using T = __nv_bfloat16;
    extern __shared__ float rotation[];   // cos[half], sin[half]
    const int token = blockIdx.x;
    const int hd = layout.head_dim, lanes_per_head = hd / 8;
    const int half = rotary_dim / 2;
    const int width = (num_heads + 2 * layout.num_groups) * hd;
    const int position = positions[token];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sine, cosine;
        sincosf(static_cast<float>(position) * inv_freq[i], &sine, &cosine);
        rotation[i] = cosine;
        rotation[half + i] = sine;
    }
    __syncthreads();
    const int units = num_heads + (write_kv ? layout.num_groups : 0);
    const int unit = threadIdx.x / lanes_per_head, chunk = threadIdx.x - unit * lanes_per_head;
    const bool active = unit < units;   // idle threads still take part in the shuffles
    const bool is_query = unit < num_heads;
    const int group = unit - num_heads;
    const float* weight = is_query ? q_weight : k_weight;
    float own[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) own[i] = 0.0f;
    if (active) {
        const uint4 raw = *reinterpret_cast<const uint4*>(qkv + static_cast<size_t>(token) * width + static_cast<size_t>(unit) * hd + chunk * 8);
        const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 two = __bfloat1622float2(pairs[i]);
            own[2 * i] = two.x;
            own[2 * i + 1] = two.y;
        }
    }
    {
        // every thread takes part in the shuffles, whether its head is normalised or not
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) sum += own[i] * own[i];
        for (int offset = 1; offset < lanes_per_head; offset <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
        const float inv = rsqrtf(sum / static_cast<float>(hd) + eps);
        if (active && weight != nullptr) {
#pragma unroll
            for (int i = 0; i < 8; ++i) own[i] = round_to<T>(round_to<T>(own[i] * inv) * round_to<T>(weight[chunk * 8 + i] + scale_offset));
        }
    }
    // rot = concat(-y[half:], y[:half]) over the first rotary_dim channels: the partner of this
    // thread's 8 channels are the 8 channels of the thread half / 8 lanes further or back.
    const bool rotates = chunk * 8 < rotary_dim;
    const bool first_half = chunk * 8 < half;
    const int partner_lane = (static_cast<int>(threadIdx.x) & 31) + (first_half ? half / 8 : -(half / 8));
    float result[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float other = __shfl_sync(0xffffffffu, own[i], rotates ? partner_lane : 0);
        result[i] = own[i];
        if (rotates) {
            const int index = (first_half ? chunk * 8 : chunk * 8 - half) + i;
            const float rotated = first_half ? -other : other;
            result[i] = own[i] * rotation[index] + rotated * rotation[half + index];
        }
    }
    if (!active) return;
    uint4 packed;
    __nv_bfloat162* packed_pairs = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int i = 0; i < 4; ++i) packed_pairs[i] = __floats2bfloat162_rn(result[2 * i], result[2 * i + 1]);
    if (is_query) {
        *reinterpret_cast<uint4*>(q_out + (static_cast<size_t>(token) * num_heads + unit) * hd + chunk * 8) = packed;
        return;
    }
    const int segment = token_segment[token];
    T* key_row = page_row(k_pages, block_table, layout, segment, position, group);
    T* value = value_column(v_pages, block_table, layout, segment, position, group);
    if (key_row == nullptr || value == nullptr) {
        if (chunk == 0) report_error(status, kBadPage);
        return;
    }
    *reinterpret_cast<uint4*>(key_row + chunk * 8) = packed;
    const uint4 v_raw =
        *reinterpret_cast<const uint4*>(qkv + static_cast<size_t>(token) * width + static_cast<size_t>(num_heads + layout.num_groups + group) * hd + chunk * 8);
    const T* v_values = reinterpret_cast<const T*>(&v_raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) value[static_cast<size_t>(chunk * 8 + i) * layout.page_size] = v_values[i];
}

// The same for steps of many tokens: one block per RUN consecutive tokens.  A thread asks for all of its
// tokens' channels before it works on the first, and where the run lies within one request at positions
// that start at a multiple of RUN, the values, which are stored transposed ([channel][row of the page]), leave
// as one store of RUN rows per channel instead of RUN stores of two bytes.
template <int RUN>
__global__ void qk_norm_rope_write_run_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                                              __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                                              const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
                                              float scale_offset, const float* __restrict__ inv_freq, int rotary_dim,
                                              const int* __restrict__ positions, const int* __restrict__ token_segment,
                                              const int* __restrict__ block_table, PagedLayout layout, int num_heads, int write_kv,
                                              int tokens, int* status) {
    static_assert(RUN == 4 || RUN == 8, "a channel's rows leave as one 8- or 16-byte store");
    using T = __nv_bfloat16;
    extern __shared__ float rotation[];   // per token of the run: cos[half], sin[half]
    const int first = blockIdx.x * RUN;
    const int count = min(RUN, tokens - first);
    const int hd = layout.head_dim, lanes_per_head = hd / 8;
    const int half = rotary_dim / 2;
    const int width = (num_heads + 2 * layout.num_groups) * hd;
    const int units = num_heads + (write_kv ? layout.num_groups : 0);
    const int unit = threadIdx.x / lanes_per_head, chunk = threadIdx.x - unit * lanes_per_head;
    const bool active = unit < units;   // idle threads still take part in the shuffles
    const bool is_query = unit < num_heads;
    const bool writes_values = active && !is_query;
    const int group = unit - num_heads;
    const float* weight = is_query ? q_weight : k_weight;
    uint4 raw[RUN], v_raw[RUN];
#pragma unroll
    for (int t = 0; t < RUN; ++t) {
        raw[t] = make_uint4(0u, 0u, 0u, 0u);
        v_raw[t] = make_uint4(0u, 0u, 0u, 0u);
        if (active && t < count) {
            const __nv_bfloat16* row = qkv + static_cast<size_t>(first + t) * width;
            raw[t] = *reinterpret_cast<const uint4*>(row + static_cast<size_t>(unit) * hd + chunk * 8);
            if (writes_values) v_raw[t] = *reinterpret_cast<const uint4*>(row + static_cast<size_t>(num_heads + layout.num_groups + group) * hd + chunk * 8);
        }
    }
    // (the loads above are on their way while the sines and cosines are worked out)
    for (int i = threadIdx.x; i < count * half; i += blockDim.x) {
        const int t = i / half, f = i - t * half;
        float sine, cosine;
        sincosf(static_cast<float>(positions[first + t]) * inv_freq[f], &sine, &cosine);
        rotation[t * rotary_dim + f] = cosine;
        rotation[t * rotary_dim + half + f] = sine;
    }
    float scale[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) scale[i] = active && weight != nullptr ? round_to<T>(weight[chunk * 8 + i] + scale_offset) : 1.0f;
    const int segment = token_segment[first];
    const int position0 = positions[first];
    // the run's values share their rows' 16-byte piece of each channel
    const bool together = count == RUN && token_segment[first + RUN - 1] == segment && positions[first + RUN - 1] == position0 + RUN - 1 &&
                          position0 % RUN == 0 && layout.page_size % RUN == 0;
    const bool rotates = chunk * 8 < rotary_dim;
    const bool first_half = chunk * 8 < half;
    const int partner_lane = (static_cast<int>(threadIdx.x) & 31) + (first_half ? half / 8 : -(half / 8));
    __syncthreads();   // the sines and cosines are there
#pragma unroll
    for (int t = 0; t < RUN; ++t) {
        float own[8];
        const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw[t]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 two = __bfloat1622float2(pairs[i]);
            own[2 * i] = two.x;
            own[2 * i + 1] = two.y;
        }
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) sum += own[i] * own[i];
        for (int offset = 1; offset < lanes_per_head; offset <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
        const float inv = rsqrtf(sum / static_cast<float>(hd) + eps);
        if (active && weight != nullptr) {
#pragma unroll
            for (int i = 0; i < 8; ++i) own[i] = round_to<T>(round_to<T>(own[i] * inv) * scale[i]);
        }
        // rot = concat(-y[half:], y[:half]) over the first rotary_dim channels: the partner of this thread's 8
        // channels are the 8 channels of the thread half / 8 lanes further or back.
        const float* turn = rotation + t * rotary_dim;
        float result[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float other = __shfl_sync(0xffffffffu, own[i], rotates ? partner_lane : 0);
            result[i] = own[i];
            if (rotates && t < count) {
                const int index = (first_half ? chunk * 8 : chunk * 8 - half) + i;
                const float rotated = first_half ? -other : other;
                result[i] = own[i] * turn[index] + rotated * turn[half + index];
            }
        }
        if (!active || t >= count) continue;
        uint4 packed;
        __nv_bfloat162* packed_pairs = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int i = 0; i < 4; ++i) packed_pairs[i] = __floats2bfloat162_rn(result[2 * i], result[2 * i + 1]);
        const int token = first + t;
        if (is_query) {
            *reinterpret_cast<uint4*>(q_out + (static_cast<size_t>(token) * num_heads + unit) * hd + chunk * 8) = packed;
            continue;
        }
        const int token_position = together ? position0 + t : positions[token];
        const int token_request = together ? segment : token_segment[token];
        T* key_row = page_row(k_pages, block_table, layout, token_request, token_position, group);
        if (key_row == nullptr) {
            if (chunk == 0) report_error(status, kBadPage);
            continue;
        }
        *reinterpret_cast<uint4*>(key_row + chunk * 8) = packed;
        if (!together) {
            T* value = value_column(v_pages, block_table, layout, token_request, token_position, group);
            if (value == nullptr) continue;
            const T* v_values = reinterpret_cast<const T*>(&v_raw[t]);
#pragma unroll
            for (int i = 0; i < 8; ++i) value[static_cast<size_t>(chunk * 8 + i) * layout.page_size] = v_values[i];
        }
    }
    if (!together || !writes_values) return;
    T* value = value_column(v_pages, block_table, layout, segment, position0, group);
    if (value == nullptr) return;   // reported with the keys
    // word w of token t holds channels 2 w (low half) and 2 w + 1; a channel's store holds tokens 0 ... RUN - 1
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const uint32_t* words[RUN];
#pragma unroll
        for (int t = 0; t < RUN; ++t) words[t] = reinterpret_cast<const uint32_t*>(&v_raw[t]);
#pragma unroll
        for (int high = 0; high < 2; ++high) {
            uint32_t column[RUN / 2];
#pragma unroll
            for (int t = 0; t < RUN / 2; ++t) column[t] = __byte_perm(words[2 * t][w], words[2 * t + 1][w], high ? 0x7632 : 0x5410);
            T* destination = value + static_cast<size_t>(chunk * 8 + 2 * w + high) * layout.page_size;
            if constexpr (RUN == 8) {
                *reinterpret_cast<uint4*>(destination) = make_uint4(column[0], column[1], column[2], column[3]);
            } else {
                *reinterpret_cast<uint2*>(destination) = make_uint2(column[0], column[1]);
            }
        }
    }
}

constexpr int kRunKernelMinTokens = 512;   // below, a block per token fills the GPU better

constexpr int kPlainChunk = 256;   // keys per softmax chunk
constexpr int kPlainThreads = 128;
constexpr int kPlainMaxDimsPerThread = 4;   // head_dim <= 512

// grid (tokens, num_heads).  The query at absolute position p sees keys j with
// max(0, p - window + 1) <= j <= p (window <= 0: all j <= p).  Scores, softmax and the
// weighted sum of values are 32-bit.
template <typename T>
__global__ void paged_attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ k_pages,
                                             const T* __restrict__ v_pages, T* __restrict__ out,
                                             const int* __restrict__ positions, const int* __restrict__ token_segment,
                                             const int* __restrict__ block_table, PagedLayout layout, int num_heads,
                                             float scale, int window, int* status) {
    extern __shared__ float shared[];
    const int hd = layout.head_dim;
    float* q_shared = shared;                    // hd
    float* scores = shared + hd;                 // kPlainChunk
    float* scratch = scores + kPlainChunk;       // 33
    const int token = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int group = head / (num_heads / layout.num_groups);
    const int segment = token_segment[token];
    const int position = positions[token];
    const int first = window > 0 ? max(0, position - window + 1) : 0;

    const T* q_row = q + (static_cast<size_t>(token) * num_heads + head) * hd;
    for (int d = tid; d < hd; d += blockDim.x) q_shared[d] = to_float(q_row[d]);
    __syncthreads();

    float acc[kPlainMaxDimsPerThread];
#pragma unroll
    for (int i = 0; i < kPlainMaxDimsPerThread; ++i) acc[i] = 0.0f;
    float running_max = -INFINITY, running_sum = 0.0f;

    for (int chunk = first; chunk <= position; chunk += kPlainChunk) {
        const int count = min(kPlainChunk, position - chunk + 1);
        float local_max = -INFINITY;
        for (int i = tid; i < count; i += blockDim.x) {
            const T* k_row = page_row(const_cast<T*>(k_pages), block_table, layout, segment, chunk + i, group);
            float s = -INFINITY;
            if (k_row == nullptr) {
                report_error(status, kBadPage);
            } else {
                float dot = 0.0f;
                for (int d = 0; d < hd; ++d) dot += q_shared[d] * to_float(k_row[d]);
                s = dot * scale;
            }
            scores[i] = s;
            local_max = fmaxf(local_max, s);
        }
        const float chunk_max = block_max(local_max, scratch);
        const float new_max = fmaxf(running_max, chunk_max);
        const float rescale = running_max == -INFINITY ? 0.0f : expf(running_max - new_max);
        float local_sum = 0.0f;
        for (int i = tid; i < count; i += blockDim.x) {
            const float p = new_max == -INFINITY ? 0.0f : expf(scores[i] - new_max);
            scores[i] = p;
            local_sum += p;
        }
        const float chunk_sum = block_sum(local_sum, scratch);   // also orders the writes to scores[]
        running_sum = running_sum * rescale + chunk_sum;
        running_max = new_max;
#pragma unroll
        for (int slot = 0; slot < kPlainMaxDimsPerThread; ++slot) {
            const int d = tid + slot * kPlainThreads;
            if (d < hd) {
                float sum = acc[slot] * rescale;
                for (int i = 0; i < count; ++i) {
                    const float p = scores[i];
                    if (p != 0.0f) {
                        const T* v_column = value_column(const_cast<T*>(v_pages), block_table, layout, segment, chunk + i, group);
                        if (v_column != nullptr) sum += p * to_float(v_column[static_cast<size_t>(d) * layout.page_size]);
                    }
                }
                acc[slot] = sum;
            }
        }
        __syncthreads();   // scores[] is rewritten by the next chunk
    }
    T* dst = out + (static_cast<size_t>(token) * num_heads + head) * hd;
    const float norm = running_sum > 0.0f ? 1.0f / running_sum : 0.0f;
#pragma unroll
    for (int slot = 0; slot < kPlainMaxDimsPerThread; ++slot) {
        const int d = tid + slot * kPlainThreads;
        if (d < hd) dst[d] = from_float<T>(acc[slot] * norm);
    }
}

}  // namespace lb

extern "C" {

int lb_qk_norm_rope_write(const void* qkv, void* q_out, void* k_pages, void* v_pages, const float* q_weight,
                          const float* k_weight, float eps, float scale_offset, const float* inv_freq, int rotary_dim,
                          const int* positions, const int* token_segment, const int* block_table, int tokens,
                          int num_heads, int num_groups, int head_dim, int page_size, int num_pages, int max_blocks,
                          int write_kv, int dtype, int* status, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (rotary_dim < 0 || rotary_dim > head_dim || rotary_dim % 2 != 0) return -2;
    lb::PagedLayout layout{page_size, num_pages, max_blocks, num_groups, head_dim};
    const bool power_of_two_head = head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128;
    const int vector_threads = (((num_heads + num_groups) * (head_dim / 8)) + 31) / 32 * 32;
    if (tokens > 64 && dtype == lb::kBFloat16 && power_of_two_head && rotary_dim % 16 == 0 && rotary_dim <= head_dim && vector_threads <= 1024 &&
        ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_pages) | reinterpret_cast<uintptr_t>(v_pages)) & 15) == 0) {
        const size_t shared = static_cast<size_t>(rotary_dim > 0 ? rotary_dim : 2) * sizeof(float);
        if (tokens >= lb::kRunKernelMinTokens) {
            constexpr int kRun = 4;
            lb::qk_norm_rope_write_run_kernel<kRun><<<(tokens + kRun - 1) / kRun, vector_threads, kRun * shared, stream>>>(
                static_cast<const __nv_bfloat16*>(qkv), static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_pages),
                static_cast<__nv_bfloat16*>(v_pages), q_weight, k_weight, eps, scale_offset, inv_freq, rotary_dim, positions, token_segment, block_table,
                layout, num_heads, write_kv, tokens, status);
            return LB_LAUNCH_RESULT();
        }
        lb::qk_norm_rope_write_vector_kernel<<<tokens, vector_threads, shared, stream>>>(
            static_cast<const __nv_bfloat16*>(qkv), static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_pages),
            static_cast<__nv_bfloat16*>(v_pages), q_weight, k_weight, eps, scale_offset, inv_freq, rotary_dim, positions, token_segment, block_table,
            layout, num_heads, write_kv, status);
        return LB_LAUNCH_RESULT();
    }
    if (tokens > 64) {
        // Many tokens: one block per token, the rotation computed once for all of its heads.
        const size_t shared = static_cast<size_t>(rotary_dim > 0 ? rotary_dim : 2) * sizeof(float);
        LB_DISPATCH_DTYPE(dtype, {
            lb::qk_norm_rope_write_token_kernel<T><<<dim3(tokens, (num_heads + num_groups + lb::kTokenKernelUnits - 1) / lb::kTokenKernelUnits), 128, shared, stream>>>(
                static_cast<const T*>(qkv), static_cast<T*>(q_out), static_cast<T*>(k_pages), static_cast<T*>(v_pages), q_weight,
                k_weight, eps, scale_offset, inv_freq, rotary_dim, positions, token_segment, block_table, layout, num_heads,
                write_kv, status);
        })
        return LB_LAUNCH_RESULT();
    }
    const dim3 grid(tokens, num_heads + num_groups);
    LB_DISPATCH_DTYPE(dtype, {
        lb::launch_overlapped(lb::qk_norm_rope_write_kernel<T>, grid, dim3(32), 0, stream,
            static_cast<const T*>(qkv), static_cast<T*>(q_out), static_cast<T*>(k_pages), static_cast<T*>(v_pages), q_weight,
            k_weight, eps, scale_offset, inv_freq, rotary_dim, positions, token_segment, block_table, layout, num_heads,
            write_kv, status);
    })
    return LB_LAUNCH_RESULT();
}

int lb_paged_attention_plain(const void* q, const void* k_pages, const void* v_pages, void* out, const int* positions,
                             const int* token_segment, const int* block_table, int tokens, int num_heads,
                             int num_groups, int head_dim, int page_size, int num_pages, int max_blocks, float scale,
                             int window, int dtype, int* status, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (head_dim > lb::kPlainThreads * lb::kPlainMaxDimsPerThread || num_heads % num_groups != 0) return -2;
    lb::PagedLayout layout{page_size, num_pages, max_blocks, num_groups, head_dim};
    const dim3 grid(tokens, num_heads);
    const size_t shared = (static_cast<size_t>(head_dim) + lb::kPlainChunk + 33) * sizeof(float);
    LB_DISPATCH_DTYPE(dtype, {
        lb::paged_attention_plain_kernel<T><<<grid, lb::kPlainThreads, shared, stream>>>(
            static_cast<const T*>(q), static_cast<const T*>(k_pages), static_cast<const T*>(v_pages), static_cast<T*>(out),
            positions, token_segment, block_table, layout, num_heads, scale, window, status);
    })
    return LB_LAUNCH_RESULT();
}

}  // extern "C"
