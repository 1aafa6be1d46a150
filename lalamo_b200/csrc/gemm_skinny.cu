// Weight-streaming matrix products for steps of up to 16 tokens (decoding):
//     Y[m, n] = sum_k X[m, k] * W[n, k]        X: [M <= 16, K] bfloat16,  W: [N, K] bfloat16
// with the step's elementwise work fused into the epilogue.  Such a product is bound by reading W
// once from HBM, so the kernel is built around that stream: a CTA owns 8 to 32 rows of W (or as
// many of each of two or three row blocks that the epilogue combines);
// its 8 warps take consecutive 32-column chunks, and every lane loads 16 contiguous
// bytes per row straight into mma.sync fragment registers (the contraction index is permuted the same way for X, which is legal since a
// dot product does not care about the order of its terms).  A CTA takes
// 8 or 16 rows and all columns.
// Accumulation is 32-bit; the warps' partial sums are added in warp order in shared memory.
//
// Epilogues:
//   kStore        Y[m, n] as bfloat16
//   kStoreFloat   Y[m, n] as float32 (logits)
//   kResidualAdd  R[m, n] += Y[m, n] on the 32-bit residual stream
//   kGated        rows n (up) and hidden + n (gate) of W: out[m, n] = up * act(gate)
//   kShortConv    rows n (B), dim + n (C), 2 dim + n (x) of W: the gated short convolution with its
//                 per-request state (see short_conv.cu for the formulas), state updated in place
#include "common.cuh"

namespace lb {

constexpr int kSkinnyWarps = 8;

enum SkinnyEpilogue : int { kStore = 0, kStoreFloat = 1, kResidualAdd = 2, kGated = 3, kShortConv = 4 };

struct SkinnyParams {
    const __nv_bfloat16* x;   // [tokens, k]
    const __nv_bfloat16* w;   // [rows, k]
    void* out;                // see the epilogues
    int tokens, k, n;         // n: output columns (rows of one row block of W)
    int row_block_stride;     // rows between the row blocks that the epilogue combines
    int activation;
    // short convolution
    __nv_bfloat16* state;             // [slots, taps - 1, n]
    const float* conv_weight;         // [n, taps]
    const float* conv_bias;           // [n] or null
    const int* token_segment;
    const int* segment_start;
    const int* segment_length;
    const int* segment_slot;
    int segments, taps, num_slots;
    int* status;
    int prefetch;   // ask for the CTA's rows of W towards L2 before waiting for the kernel before this one
};

__device__ __forceinline__ void mma_16816_skinny(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float skinny_activate(float v, int activation) {
    if (activation == 0) return v / (1.0f + expf(-v));
    if (activation == 1) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
    return v;
}

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// Tokens are the 16 rows of the mma tile (rows 8..15 are left out when at most 8 tokens run), rows
// of W its 8 columns.  TILES: row blocks of W per CTA (1; 2 for kGated; 3 for kShortConv).
// RG: groups of 8 rows of W per row block and CTA.  WIDE: more than 8 tokens.
template <int TILES, int RG, bool WIDE, int EPILOGUE>
__global__ void __launch_bounds__(kSkinnyWarps * 32, TILES == 3 ? 1 : 2)
gemm_skinny_kernel(const SkinnyParams p) {
    constexpr int ROWS = 8 * RG;        // rows of each row block this CTA computes
    constexpr int TOKENS = WIDE ? 16 : 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * ROWS;
    const int chunks = p.k / 32;

    float acc[TILES][RG][4];
#pragma unroll
    for (int tile = 0; tile < TILES; ++tile)
#pragma unroll
        for (int r = 0; r < RG; ++r) acc[tile][r][0] = acc[tile][r][1] = acc[tile][r][2] = acc[tile][r][3] = 0.0f;

    const __nv_bfloat16* w_rows[TILES][RG];
#pragma unroll
    for (int tile = 0; tile < TILES; ++tile)
#pragma unroll
        for (int r = 0; r < RG; ++r)
            w_rows[tile][r] = p.w + (static_cast<size_t>(tile) * p.row_block_stride + row0 + 8 * r + g) * p.k + 8 * t;
    // This kernel may have been started before the one that produces X has finished: ask for this CTA's
    // rows of W, which nobody writes, to be brought to L2 meanwhile, and only then wait for X.  One bulk
    // prefetch per row (k * 2 bytes, a multiple of 16): a prefetch per 128-byte line took a CTA 1.7 us to
    // issue for K = 8192.  Where the predecessor does not let this kernel start early (p.prefetch == 0)
    // there is nothing to wait for, and a prefetch would only stand in the way of the first loads.
    allow_next_kernel();
    if (p.prefetch) {
        const unsigned bytes = static_cast<unsigned>(p.k) * 2u;
        for (int row = threadIdx.x; row < TILES * ROWS; row += blockDim.x) {
            const int tile = row / ROWS, local = row - tile * ROWS;
            const __nv_bfloat16* source = p.w + (static_cast<size_t>(tile) * p.row_block_stride + row0 + local) * p.k;
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(source), "r"(bytes) : "memory");
        }
    }
    wait_for_previous_kernel();
    const bool low_valid = g < p.tokens, high_valid = WIDE && g + 8 < p.tokens;
    const __nv_bfloat16* x_low = p.x + static_cast<size_t>(low_valid ? g : 0) * p.k + 8 * t;
    const __nv_bfloat16* x_high = p.x + static_cast<size_t>(high_valid ? g + 8 : 0) * p.k + 8 * t;

    // Chunks whose loads are issued together.  A small product is bound by latency unless (nearly) all
    // of the matrix is in flight at once, so the leanest variant loads eight chunks per lane at a time.
    constexpr int UNROLL = (TILES * RG == 1) ? 8 : 4;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int chunk = warp; chunk < chunks; chunk += kSkinnyWarps * UNROLL) {
        uint4 wb[UNROLL][TILES][RG];
        uint4 xa[UNROLL][2];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int c = chunk + u * kSkinnyWarps;
            if (chunk + u * kSkinnyWarps < chunks) {
#pragma unroll
                for (int tile = 0; tile < TILES; ++tile)
#pragma unroll
                    for (int r = 0; r < RG; ++r) wb[u][tile][r] = __ldcs(reinterpret_cast<const uint4*>(w_rows[tile][r] + c * 32));
                xa[u][0] = low_valid ? __ldg(reinterpret_cast<const uint4*>(x_low + c * 32)) : zero;
                xa[u][1] = high_valid ? __ldg(reinterpret_cast<const uint4*>(x_high + c * 32)) : zero;
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            if (chunk + u * kSkinnyWarps < chunks) {
#pragma unroll
                for (int tile = 0; tile < TILES; ++tile) {
#pragma unroll
                    for (int r = 0; r < RG; ++r) {
                        // 32 columns = two k16 blocks: a lane's bytes 0-7 feed the first, 8-15 the second.
                        mma_16816_skinny(acc[tile][r], xa[u][0].x, xa[u][1].x, xa[u][0].y, xa[u][1].y, wb[u][tile][r].x, wb[u][tile][r].y);
                        mma_16816_skinny(acc[tile][r], xa[u][0].z, xa[u][1].z, xa[u][0].w, xa[u][1].w, wb[u][tile][r].z, wb[u][tile][r].w);
                    }
                }
            }
        }
    }

    // Add the warps' partial sums in warp order.  partial[warp][tile][row][token]
    __shared__ float partial[kSkinnyWarps][TILES][ROWS][TOKENS + 1];
#pragma unroll
    for (int tile = 0; tile < TILES; ++tile) {
#pragma unroll
        for (int r = 0; r < RG; ++r) {
            partial[warp][tile][8 * r + 2 * t][g] = acc[tile][r][0];
            partial[warp][tile][8 * r + 2 * t + 1][g] = acc[tile][r][1];
            if (WIDE) {
                partial[warp][tile][8 * r + 2 * t][g + 8] = acc[tile][r][2];
                partial[warp][tile][8 * r + 2 * t + 1][g + 8] = acc[tile][r][3];
            }
        }
    }
    __syncthreads();
    __shared__ float total[TILES][ROWS][TOKENS + 1];
    for (int index = threadIdx.x; index < TILES * ROWS * TOKENS; index += blockDim.x) {
        const int token = index % TOKENS, row = (index / TOKENS) % ROWS, tile = index / (TOKENS * ROWS);
        float sum = 0.0f;
#pragma unroll
        for (int w = 0; w < kSkinnyWarps; ++w) sum += partial[w][tile][row][token];
        total[tile][row][token] = sum;
    }
    __syncthreads();

    if constexpr (EPILOGUE == kStore || EPILOGUE == kStoreFloat || EPILOGUE == kResidualAdd || EPILOGUE == kGated) {
        // Threads walk rows fastest so that stores of one token are contiguous.
        for (int index = threadIdx.x; index < ROWS * TOKENS; index += blockDim.x) {
            const int row = index % ROWS, token = index / ROWS;
            if (token >= p.tokens) continue;
            const size_t where = static_cast<size_t>(token) * p.n + row0 + row;
            const float value = total[0][row][token];
            if constexpr (EPILOGUE == kStore) {
                static_cast<__nv_bfloat16*>(p.out)[where] = __float2bfloat16_rn(value);
            } else if constexpr (EPILOGUE == kStoreFloat) {
                static_cast<float*>(p.out)[where] = value;
            } else if constexpr (EPILOGUE == kResidualAdd) {
                static_cast<float*>(p.out)[where] += round_bf16(value);
            } else {
                const float up = round_bf16(value), gate = round_bf16(total[1][row][token]);
                static_cast<__nv_bfloat16*>(p.out)[where] = __float2bfloat16_rn(up * round_bf16(skinny_activate(gate, p.activation)));
            }
        }
    } else {
        // Short convolution over this CTA's channels: total[0] = B, total[1] = C, total[2] = x.
        __shared__ float gated_input[TOKENS][ROWS];
        for (int index = threadIdx.x; index < ROWS * TOKENS; index += blockDim.x) {
            const int row = index % ROWS, token = index / ROWS;
            gated_input[token][row] = round_bf16(round_bf16(total[0][row][token]) * round_bf16(total[2][row][token]));
        }
        __syncthreads();
        const int history = p.taps - 1;
        for (int index = threadIdx.x; index < ROWS * TOKENS; index += blockDim.x) {
            const int row = index % ROWS, token = index / ROWS;
            if (token >= p.tokens) continue;
            const int channel = row0 + row;
            const int segment = p.token_segment[token];
            const int start = p.segment_start[segment];
            const int j = token - start;
            const int slot = p.segment_slot[segment];
            if (slot < 0 || slot >= p.num_slots) {
                report_error(p.status, kBadSlot);
                continue;
            }
            const __nv_bfloat16* slot_state = p.state + static_cast<size_t>(slot) * history * p.n;
            const float* taps = p.conv_weight + static_cast<size_t>(channel) * p.taps;
            float sum = 0.0f;
            for (int tap = 0; tap < p.taps; ++tap) {
                const int i = j + tap - history;
                const float value = i >= 0 ? gated_input[start + i][row] : __bfloat162float(slot_state[static_cast<size_t>(history + i) * p.n + channel]);
                sum += taps[tap] * value;
            }
            const float conv = round_bf16(sum + (p.conv_bias ? p.conv_bias[channel] : 0.0f));
            static_cast<__nv_bfloat16*>(p.out)[static_cast<size_t>(token) * p.n + channel] = __float2bfloat16_rn(round_bf16(total[1][row][token]) * conv);
        }
        __syncthreads();   // every read of the old state is done
        for (int index = threadIdx.x; index < ROWS * p.segments; index += blockDim.x) {
            const int row = index % ROWS, segment = index / ROWS;
            const int channel = row0 + row;
            const int slot = p.segment_slot[segment];
            if (slot < 0 || slot >= p.num_slots) continue;
            const int start = p.segment_start[segment], length = p.segment_length[segment];
            __nv_bfloat16* slot_state = p.state + static_cast<size_t>(slot) * history * p.n;
            for (int r = 0; r < history; ++r) {   // row r <- hist[length + r]; sources lie above r
                const int i = length + r;
                slot_state[static_cast<size_t>(r) * p.n + channel] =
                    i < history ? slot_state[static_cast<size_t>(i) * p.n + channel] : __float2bfloat16_rn(gated_input[start + i - history][row]);
            }
        }
    }
}


template <int TILES, int EPILOGUE>
int launch_skinny(const SkinnyParams& p, cudaStream_t stream) {
    const bool wide = p.tokens > 8;
    // 16 rows per CTA when that still fills the GPU twice over, else 8.
    const bool two_groups = TILES == 1 && p.n % 16 == 0 && p.n / 16 >= 2 * multiprocessor_count();
    const dim3 block(kSkinnyWarps * 32);
    if constexpr (TILES == 1) {
        if (two_groups) {
            return wide ? static_cast<int>(launch_overlapped(gemm_skinny_kernel<1, 2, true, EPILOGUE>, dim3(p.n / 16), block, 0, stream, p))
                        : static_cast<int>(launch_overlapped(gemm_skinny_kernel<1, 2, false, EPILOGUE>, dim3(p.n / 16), block, 0, stream, p));
        }
    }
    return wide ? static_cast<int>(launch_overlapped(gemm_skinny_kernel<TILES, 1, true, EPILOGUE>, dim3(p.n / 8), block, 0, stream, p))
                : static_cast<int>(launch_overlapped(gemm_skinny_kernel<TILES, 1, false, EPILOGUE>, dim3(p.n / 8), block, 0, stream, p));
}

}  // namespace lb

extern "C" {

// Returns 0, a CUDA error, or -2 when the sizes are not the kernel's (1..16 tokens, k % 32 == 0,
// n % 8 == 0, 16-byte aligned rows).
int lb_gemm_skinny(const void* x, const void* w, void* out, int tokens, int k, int n, int epilogue, int activation,
                   void* state, const float* conv_weight, const float* conv_bias, const int* token_segment,
                   const int* segment_start, const int* segment_length, const int* segment_slot, int segments, int taps,
                   int num_slots, int prefetch, int* status, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (tokens < 1 || tokens > 16 || k % 32 != 0 || n % 8 != 0 || k < 32) return -2;
    lb::SkinnyParams p;
    p.x = static_cast<const __nv_bfloat16*>(x);
    p.w = static_cast<const __nv_bfloat16*>(w);
    p.out = out;
    p.tokens = tokens;
    p.k = k;
    p.n = n;
    p.row_block_stride = n;
    p.activation = activation;
    p.state = static_cast<__nv_bfloat16*>(state);
    p.conv_weight = conv_weight;
    p.conv_bias = conv_bias;
    p.token_segment = token_segment;
    p.segment_start = segment_start;
    p.segment_length = segment_length;
    p.segment_slot = segment_slot;
    p.segments = segments;
    p.taps = taps;
    p.num_slots = num_slots;
    p.status = status;
    p.prefetch = prefetch && (reinterpret_cast<uintptr_t>(w) & 15) == 0 ? 1 : 0;
    switch (epilogue) {
        case lb::kStore: return lb::launch_skinny<1, lb::kStore>(p, stream);
        case lb::kStoreFloat: return lb::launch_skinny<1, lb::kStoreFloat>(p, stream);
        case lb::kResidualAdd: return lb::launch_skinny<1, lb::kResidualAdd>(p, stream);
        case lb::kGated: return lb::launch_skinny<2, lb::kGated>(p, stream);
        case lb::kShortConv:
            if (taps < 1 || segments < 1 || segments > tokens) return -2;
            return lb::launch_skinny<3, lb::kShortConv>(p, stream);
        default: return -2;
    }
}

}  // extern "C"
