// Paged attention for tokens that attend alone (decoding, and short portions): split over the
// keys, tensor-core products, every lane copying just the bytes of its own operand fragments.
//
// One CTA handles (split of the keys, K/V head + up to 16 of its query heads, token).  Each of its
// warps walks 16-key blocks of the split, two at a time:
//   S[heads x 16 keys] = Q K^T      mma.sync m16n8k16, A = Q (rows: query heads of the group), B = K rows
//   online softmax in 32-bit (base 2, ex2.approx), one update per two blocks
//   O[heads x hd]     += P V        A = P (the accumulators of S, rounded to bfloat16), B = V^T rows
// The contraction index of a matrix product may be permuted if both operands agree, which is
// used twice so that every global read is contiguous and a lane needs no other lane's bytes:
//   * channels: lane t of a quad owns channels [t*hd/4, (t+1)*hd/4) of its key row (and of Q);
//   * keys: column n of 8-key block b stands for key 4*(n/2) + 2*b + n%2 of the 16, so that lane t
//     holds probabilities of keys 4t..4t+3, which are contiguous in the transposed value page.
// Keys are [page][row][group][hd]; values are transposed, [page][group][hd][row]; page_size % 16 == 0.
// Partial results (max, sum, unnormalised output per split) go to scratch; a second kernel merges
// them in split order, so the result does not depend on the batch or on the grid.
#include "common.cuh"

namespace lb {

constexpr int kDecodeWarps = 4;

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 2^x by the hardware's approximation (two units in the last place of float32); 2^-inf = 0.
__device__ __forceinline__ float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float low, float high) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<const uint32_t*>(&pair);
}

constexpr float kDecodeMaxSlack = 8.0f;   // how far a row's maximum may outgrow its reference exponent (base 2)

struct DecodeParams {
    const __nv_bfloat16* q;         // [tokens, heads, hd]
    const __nv_bfloat16* k_pages;   // [pages, page_size, groups, hd]
    const __nv_bfloat16* v_pages;   // [pages, groups, hd, page_size]
    __nv_bfloat16* out;             // [tokens, heads, hd]: written by this kernel itself when there is one split
    float* partial_out;             // [tokens, heads, splits, hd]
    float* partial_stats;           // [tokens, heads, splits, 2]  (max in base-2 units, sum)
    const int* positions;
    const int* token_segment;
    const int* block_table;
    const int* token_list;          // the tokens to run (null: all, in order); partials are indexed by list place
    int num_heads, num_groups, page_size, num_pages, max_blocks;
    int splits, blocks_per_split;   // in units of 16 keys
    int window;
    float scale_log2;               // scale * log2(e)
    int* status;
    // >= 0: the kernel is launched to start before the kernel before it has finished, and the newest `fresh_keys`
    // positions a token sees may still be written by that kernel; it reads the older ones while it waits.
    int fresh_keys;
};

// The page that holds 16-key block `key_block` of the request, or -1, and the block's first row in it.
__device__ __forceinline__ int decode_page_of(const DecodeParams& p, int segment, int key_block, int& in_page) {
    const int table_column = key_block * 16 / p.page_size;
    in_page = key_block * 16 - table_column * p.page_size;
    const int page = table_column < p.max_blocks ? p.block_table[static_cast<size_t>(segment) * p.max_blocks + table_column] : -1;
    return page >= 0 && page < p.num_pages ? page : -1;
}

// What a lane's copies of a block have in common, worked out once per kernel: the addresses of a block's
// fragments are these plus the page's and the row's offsets (the division by the page size and the
// multiplications by the layout's strides took a third of the kernel's instructions when they were
// done for every block).
struct DecodeLaneSources {
    const __nv_bfloat16* keys[2];   // this lane's two key rows of a block, at row 0 of page 0
    const __nv_bfloat16* values;    // this lane's first value row, at key 0 of page 0
    size_t key_page_stride, value_page_stride;   // elements from page to page
    int key_row_stride;             // elements from key to key
    int value_step;                 // elements from a lane's value row to its next (8 channels on)
};

template <int HD>
__device__ __forceinline__ DecodeLaneSources decode_lane_sources(const DecodeParams& p, int group, int lane) {
    const int g = lane >> 2, t = lane & 3;
    DecodeLaneSources sources;
    sources.key_row_stride = p.num_groups * HD;
    sources.key_page_stride = static_cast<size_t>(p.page_size) * sources.key_row_stride;
    sources.value_page_stride = static_cast<size_t>(p.num_groups) * HD * p.page_size;
    sources.value_step = 8 * p.page_size;
#pragma unroll
    for (int b = 0; b < 2; ++b) {
        const int key = 4 * (g >> 1) + 2 * b + (g & 1);
        sources.keys[b] = p.k_pages + static_cast<size_t>(key) * sources.key_row_stride + group * HD + t * (HD / 4);
    }
    sources.values = p.v_pages + (static_cast<size_t>(group) * HD + g) * p.page_size + 4 * t;
    return sources;
}

// Each warp keeps a ring of stages in shared memory, filled by asynchronous copies: a lane copies
// exactly the bytes of its own fragments (16 or 8 at a time, slot by slot, the lanes of a slot side by
// side) and later reads them back itself, so that no lane waits for another.  What the ring buys is
// depth: kStages - 1 blocks of 16 keys on their way per warp instead of the one that registers can hold.
template <int HD>
struct DecodeRing {
    static constexpr int kStageBytes = HD * 64;   // 16 keys and 16 values of HD channels
    static constexpr int kStages = 3;   // three blocks per warp on their way or in use; 48 KB per CTA at head size 64: four CTAs per SM
    static constexpr int kWarpBytes = kStages * kStageBytes;
    static constexpr int kBytes = kDecodeWarps * kWarpBytes;
    static_assert(16 * (HD + 1) * 4 <= kWarpBytes, "a warp's partial output fits its ring when the keys are done");
};

__device__ __forceinline__ void async_copy_16(void* shared_destination, const void* source) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(shared_destination))), "l"(source)
                 : "memory");
}

__device__ __forceinline__ void async_copy_8(void* shared_destination, const void* source) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(shared_destination))), "l"(source)
                 : "memory");
}

// Starts the copies of a 16-key block (rows `in_page`.. of `page`; page -1: zeros) into `stage`.
template <int HD>
__device__ __forceinline__ void issue_fragments(unsigned char* stage, const DecodeLaneSources& sources, int page, int in_page, int lane, bool& bad) {
    unsigned char* keys = stage;
    unsigned char* values = stage + HD * 32;
    if (page < 0) {
        bad = true;
        for (int i = 0; i < HD / 8; ++i) {   // HD * 64 bytes = HD / 8 rounds of 32 lanes x 16 bytes
            *reinterpret_cast<uint4*>(stage + (i * 32 + lane) * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        return;
    }
    const size_t key_offset = page * sources.key_page_stride + static_cast<size_t>(in_page) * sources.key_row_stride;
#pragma unroll
    for (int b = 0; b < 2; ++b) {
        const __nv_bfloat16* row = sources.keys[b] + key_offset;
        if constexpr (HD % 32 == 0) {
#pragma unroll
            for (int j = 0; j < HD / 32; ++j) async_copy_16(keys + ((b * (HD / 32) + j) * 32 + lane) * 16, reinterpret_cast<const uint4*>(row) + j);
        } else {
#pragma unroll
            for (int j = 0; j < HD / 16; ++j) async_copy_8(keys + ((b * (HD / 16) + j) * 32 + lane) * 8, reinterpret_cast<const uint2*>(row) + j);
        }
    }
    const __nv_bfloat16* source = sources.values + page * sources.value_page_stride + in_page;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        async_copy_8(values + (n * 32 + lane) * 8, source);
        source += sources.value_step;
    }
}

// Reads this lane's key fragments of a stage whose copies have arrived: k[8-key block][channel block][b0, b1].
template <int HD>
__device__ __forceinline__ void read_key_fragments(uint32_t (&k)[2][HD / 16][2], const unsigned char* stage, int lane) {
#pragma unroll
    for (int b = 0; b < 2; ++b) {
        if constexpr (HD % 32 == 0) {
#pragma unroll
            for (int j = 0; j < HD / 32; ++j) {
                const uint4 loaded = *reinterpret_cast<const uint4*>(stage + ((b * (HD / 32) + j) * 32 + lane) * 16);
                k[b][2 * j][0] = loaded.x;
                k[b][2 * j][1] = loaded.y;
                k[b][2 * j + 1][0] = loaded.z;
                k[b][2 * j + 1][1] = loaded.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < HD / 16; ++j) {
                const uint2 loaded = *reinterpret_cast<const uint2*>(stage + ((b * (HD / 16) + j) * 32 + lane) * 8);
                k[b][j][0] = loaded.x;
                k[b][j][1] = loaded.y;
            }
        }
    }
}

// The same for the values: v[channel block of 8][b0, b1].
template <int HD>
__device__ __forceinline__ void read_value_fragments(uint32_t (&v)[HD / 8][2], const unsigned char* stage, int lane) {
    const unsigned char* values = stage + HD * 32;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        const uint2 loaded = *reinterpret_cast<const uint2*>(values + (n * 32 + lane) * 8);
        v[n][0] = loaded.x;
        v[n][1] = loaded.y;
    }
}

// grid (splits, groups * row_tiles, tokens), kDecodeWarps warps.
template <int HD>
__global__ void __launch_bounds__(kDecodeWarps * 32, HD <= 64 ? 4 : 1)   // head size 64: 128 registers, four CTAs per SM
attention_decode_kernel(const DecodeParams p) {
    const int split = blockIdx.x, place = blockIdx.z;
    const int token = p.token_list ? p.token_list[place] : place;
    const int heads_per_group = p.num_heads / p.num_groups;
    const int row_tiles = (heads_per_group + 15) / 16;
    const int group = blockIdx.y / row_tiles, row_tile = blockIdx.y - group * row_tiles;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int position = p.positions[token];
    const int segment = p.token_segment[token];
    const int first_visible = p.window > 0 ? max(0, position - p.window + 1) : 0;
    const int first_block = first_visible / 16, last_block = position / 16;
    const int begin = first_block + split * p.blocks_per_split;
    const int end = min(begin + p.blocks_per_split, last_block + 1);
    const int rows_here = min(16, heads_per_group - row_tile * 16);
    const int head_base = group * heads_per_group + row_tile * 16;

    uint32_t q_frag[HD / 16][4];
    float out[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) out[n][0] = out[n][1] = out[n][2] = out[n][3] = 0.0f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
    bool bad = false;

    // The block table is read 32 blocks of this warp at a time (lane i: the warp's i-th block from
    // `table_first`) and handed round by shuffles: a block's keys do not wait for a table read of their own.
    using Ring = DecodeRing<HD>;
    extern __shared__ __align__(16) unsigned char ring_memory[];
    unsigned char* ring = ring_memory + warp * Ring::kWarpBytes;
    const int count = end > begin + warp ? (end - begin - warp + kDecodeWarps - 1) / kDecodeWarps : 0;   // this warp's blocks: begin + warp + 4 i
    const DecodeLaneSources sources = decode_lane_sources<HD>(p, group, lane);
    int table_first = 0;
    int lane_in_page = 0;
    int lane_page = lane < count ? decode_page_of(p, segment, begin + warp + kDecodeWarps * lane, lane_in_page) : -1;
    int issued = 0, issue_stage = 0;   // issue_stage = issued % kStages, kept by hand (the modulo costs instructions in every turn)
    // Starts the copies of this warp's next block, if there is one; a group is committed either way.
    auto issue_next = [&]() {
        if (issued < count) {
            if (issued - table_first == 32) {
                table_first = issued;
                lane_page = issued + lane < count ? decode_page_of(p, segment, begin + warp + kDecodeWarps * (issued + lane), lane_in_page) : -1;
            }
            issue_fragments<HD>(ring + issue_stage * Ring::kStageBytes, sources, __shfl_sync(0xffffffffu, lane_page, issued - table_first),
                                __shfl_sync(0xffffffffu, lane_in_page, issued - table_first), lane, bad);
            ++issued;
            issue_stage = issue_stage + 1 == Ring::kStages ? 0 : issue_stage + 1;
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    // Launched to start early (fresh_keys >= 0): the blocks of keys that the kernel before this one cannot be
    // writing are asked for at once, and the queries, which it does write, only when it is done.
    int started = 0;
    if (p.fresh_keys >= 0) {
        const int first_fresh_block = max(0, position - p.fresh_keys + 1) / 16;
        for (; started < Ring::kStages; ++started) {
            if (issued < count && begin + warp + kDecodeWarps * issued >= first_fresh_block) break;
            issue_next();
        }
        wait_for_previous_kernel();
    }
    // Q fragments of rows g and g + 8 (zero beyond the group's heads), channels permuted like K's.
#pragma unroll
    for (int j = 0; j < HD / 16; ++j) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = g + 8 * half;
            uint2 loaded = make_uint2(0u, 0u);
            if (row < rows_here) {
                const __nv_bfloat16* src = p.q + (static_cast<size_t>(token) * p.num_heads + head_base + row) * HD + t * (HD / 4) + 4 * j;
                loaded = *reinterpret_cast<const uint2*>(src);
            }
            q_frag[j][half] = loaded.x;       // a0 (row g) / a1 (row g + 8): logical k = 2t, 2t+1
            q_frag[j][2 + half] = loaded.y;   // a2 / a3: logical k = 2t+8, 2t+9
        }
    }

    for (int stage = started; stage < Ring::kStages; ++stage) issue_next();
    // Two of the warp's blocks at a time share one softmax update (one new maximum, one rescaling of
    // the output); the ring is refilled at the end of the turn, when both have been read.
    int read_stage = 0;   // index % kStages
#pragma unroll 1
    for (int index = 0; index < count; index += 2) {
        const bool two = index + 1 < count;
        const int blocks[2] = {begin + warp + kDecodeWarps * index, begin + warp + kDecodeWarps * (index + 1)};
        const int next_stage = read_stage + 1 == Ring::kStages ? 0 : read_stage + 1;
        const unsigned char* stages[2] = {ring + read_stage * Ring::kStageBytes, ring + next_stage * Ring::kStageBytes};
        read_stage = next_stage + 1 == Ring::kStages ? 0 : next_stage + 1;
        asm volatile("cp.async.wait_group %0;\n" ::"n"(Ring::kStages - 2) : "memory");   // all but the newest kStages - 2 groups: both blocks are here
        float s[2][2][4];
#pragma unroll
        for (int which = 0; which < 2; ++which) {
#pragma unroll
            for (int b = 0; b < 2; ++b) s[which][b][0] = s[which][b][1] = s[which][b][2] = s[which][b][3] = which == 1 && !two ? -INFINITY : 0.0f;
            if (which == 0 || two) {
                uint32_t k[2][HD / 16][2];
                read_key_fragments<HD>(k, stages[which], lane);
#pragma unroll
                for (int b = 0; b < 2; ++b) {
#pragma unroll
                    for (int j = 0; j < HD / 16; ++j) mma_16816(s[which][b], q_frag[j], k[b][j][0], k[b][j][1]);
                }
            }
        }
        // Lane t holds keys 4t + 2b + {0, 1} of a block for rows g (s[.][b][0..1]) and g + 8 (s[.][b][2..3]).
        // Only the first and the last block of the visible range hold keys that must not count.
        bool edge[2];
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            edge[which] = (which == 0 || two) && (blocks[which] == first_block || blocks[which] == last_block);
            if (edge[which]) {
#pragma unroll
                for (int b = 0; b < 2; ++b) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int key = blocks[which] * 16 + 4 * t + 2 * b + (c & 1);
                        if (key < first_visible || key > position) s[which][b][c] = -INFINITY;
                    }
                }
            }
        }
        float rescale[2], shift[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float pair_max = fmaxf(fmaxf(fmaxf(s[0][0][2 * r], s[0][0][2 * r + 1]), fmaxf(s[0][1][2 * r], s[0][1][2 * r + 1])),
                                   fmaxf(fmaxf(s[1][0][2 * r], s[1][0][2 * r + 1]), fmaxf(s[1][1][2 * r], s[1][1][2 * r + 1])));
            pair_max = fmaxf(pair_max, __shfl_xor_sync(0xffffffffu, pair_max, 1));
            pair_max = fmaxf(pair_max, __shfl_xor_sync(0xffffffffu, pair_max, 2));
            // row_max is the exponent the row's terms are taken relative to.  It follows the row's maximum only
            // when that has outgrown it by more than 2^8: a warp sees few blocks, and with the true maximum
            // the 32 output values of a lane were rescaled in four turns of five.
            const float top = pair_max * p.scale_log2;   // the scale is positive
            const float new_max = top > row_max[r] + kDecodeMaxSlack ? top : row_max[r];
            shift[r] = new_max == -INFINITY ? 0.0f : new_max;   // a row that has seen no key yet: every term below is 2^-inf = 0
            rescale[r] = exp2_approx(row_max[r] - shift[r]);
            row_max[r] = new_max;
        }
        float partial_sum[2] = {0.0f, 0.0f};
        uint32_t p_frag[2][4];
#pragma unroll
        for (int which = 0; which < 2; ++which) {
#pragma unroll
            for (int b = 0; b < 2; ++b) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    s[which][b][c] = exp2_approx(fmaf(s[which][b][c], p.scale_log2, -shift[c >> 1]));
                    partial_sum[c >> 1] += s[which][b][c];
                }
            }
            p_frag[which][0] = pack_bf16(s[which][0][0], s[which][0][1]);   // row g,     logical k 2t, 2t+1   = keys 4t, 4t+1
            p_frag[which][1] = pack_bf16(s[which][0][2], s[which][0][3]);   // row g + 8
            p_frag[which][2] = pack_bf16(s[which][1][0], s[which][1][1]);   // row g,     logical k 2t+8, 2t+9 = keys 4t+2, 4t+3
            p_frag[which][3] = pack_bf16(s[which][1][2], s[which][1][3]);   // row g + 8
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) row_sum[r] = row_sum[r] * rescale[r] + partial_sum[r];
        if (!__all_sync(0xffffffffu, rescale[0] == 1.0f && rescale[1] == 1.0f)) {
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) {
                out[n][0] *= rescale[0];
                out[n][1] *= rescale[0];
                out[n][2] *= rescale[1];
                out[n][3] *= rescale[1];
            }
        }
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            if (which == 0 || two) {
                uint32_t v[HD / 8][2];
                read_value_fragments<HD>(v, stages[which], lane);
                if (edge[which]) {
                    // Rows outside [first visible key, own position] hold whatever was left there (after the
                    // position: an earlier owner of the page's data, possibly not even finite): a zero
                    // probability does not silence them in the product, so clear those values.  Lane t
                    // holds keys 4t..4t+3 in v[n][0] (two) and v[n][1] (two).
                    uint32_t mask[2];
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int low = blocks[which] * 16 + 4 * t + 2 * i, high = low + 1;
                        mask[i] = ((low >= first_visible && low <= position) ? 0x0000ffffu : 0u) |
                                  ((high >= first_visible && high <= position) ? 0xffff0000u : 0u);
                    }
#pragma unroll
                    for (int n = 0; n < HD / 8; ++n) {
                        v[n][0] &= mask[0];
                        v[n][1] &= mask[1];
                    }
                }
#pragma unroll
                for (int n = 0; n < HD / 8; ++n) mma_16816(out[n], p_frag[which], v[n][0], v[n][1]);
            }
        }
        issue_next();
        issue_next();
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    if (bad && lane == 0) report_error(p.status, kBadPage);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
    }

    // Merge the warps of this CTA in warp order (shared memory), then write the split's partial.
    // A warp's partial output goes where its ring was (its own copies have all arrived).
    __shared__ float shared_max[kDecodeWarps][16], shared_sum[kDecodeWarps][16];
    auto shared_out = [&](int w, int row, int d) -> float& { return reinterpret_cast<float*>(ring_memory + w * Ring::kWarpBytes)[row * (HD + 1) + d]; };
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        shared_out(warp, g, 8 * n + 2 * t) = out[n][0];
        shared_out(warp, g, 8 * n + 2 * t + 1) = out[n][1];
        shared_out(warp, g + 8, 8 * n + 2 * t) = out[n][2];
        shared_out(warp, g + 8, 8 * n + 2 * t + 1) = out[n][3];
    }
    if (t == 0) {
        shared_max[warp][g] = row_max[0];
        shared_max[warp][g + 8] = row_max[1];
        shared_sum[warp][g] = row_sum[0];
        shared_sum[warp][g + 8] = row_sum[1];
    }
    __syncthreads();
    for (int index = threadIdx.x; index < rows_here * HD; index += blockDim.x) {
        const int row = index / HD, d = index - row * HD;
        float merged_max = -INFINITY;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; ++w) merged_max = fmaxf(merged_max, shared_max[w][row]);
        float value = 0.0f, sum = 0.0f;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; ++w) {
            const float weight = shared_max[w][row] == -INFINITY ? 0.0f : exp2f(shared_max[w][row] - merged_max);
            value += shared_out(w, row, d) * weight;
            sum += shared_sum[w][row] * weight;
        }
        if (p.splits == 1) {
            // all of the token's keys were this CTA's: what the merge kernel would make of the one partial
            p.out[(static_cast<size_t>(token) * p.num_heads + head_base + row) * HD + d] = __float2bfloat16_rn(sum > 0.0f ? value / sum : 0.0f);
            continue;
        }
        const size_t slot = (static_cast<size_t>(place) * p.num_heads + head_base + row) * p.splits + split;
        p.partial_out[slot * HD + d] = value;
        if (d == 0) {
            p.partial_stats[slot * 2] = merged_max;
            p.partial_stats[slot * 2 + 1] = sum;
        }
    }
}

// grid (heads, tokens); merges the splits in order and normalises.  The partials of up to eight
// splits are asked for together (one after the other, every split would cost a trip to L2).
template <int HD>
__global__ void attention_decode_merge_kernel(const float* __restrict__ partial_out, const float* __restrict__ partial_stats,
                                              __nv_bfloat16* __restrict__ out, const int* __restrict__ token_list, int num_heads, int splits) {
    allow_next_kernel();   // the out-projection that follows may start pulling its weights towards L2
    const int head = blockIdx.x, place = blockIdx.y;
    const int token = token_list ? token_list[place] : place;
    const size_t base = (static_cast<size_t>(place) * num_heads + head) * splits;
    constexpr int kBatch = 8;
    float merged_max = -INFINITY;
    for (int first = 0; first < splits; first += kBatch) {
        float maxima[kBatch];
#pragma unroll
        for (int i = 0; i < kBatch; ++i) maxima[i] = first + i < splits ? partial_stats[(base + first + i) * 2] : -INFINITY;
#pragma unroll
        for (int i = 0; i < kBatch; ++i) merged_max = fmaxf(merged_max, maxima[i]);
    }
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float value = 0.0f, sum = 0.0f;
        for (int first = 0; first < splits; first += kBatch) {
            float maxima[kBatch], sums[kBatch], values[kBatch];
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
                const bool here = first + i < splits;
                maxima[i] = here ? partial_stats[(base + first + i) * 2] : -INFINITY;
                sums[i] = here ? partial_stats[(base + first + i) * 2 + 1] : 0.0f;
                values[i] = here ? partial_out[(base + first + i) * HD + d] : 0.0f;
            }
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {   // in split order
                const float weight = maxima[i] == -INFINITY ? 0.0f : exp2f(maxima[i] - merged_max);
                value += values[i] * weight;
                sum += sums[i] * weight;
            }
        }
        out[(static_cast<size_t>(token) * num_heads + head) * HD + d] = __float2bfloat16_rn(sum > 0.0f ? value / sum : 0.0f);
    }
}

template <int HD>
int launch_decode(const DecodeParams& p, __nv_bfloat16* out, int tokens, cudaStream_t stream) {
    const int heads_per_group = p.num_heads / p.num_groups;
    const int row_tiles = (heads_per_group + 15) / 16;
    const dim3 grid(p.splits, p.num_groups * row_tiles, tokens);
    auto kernel = attention_decode_kernel<HD>;
    static OncePerDevice configured;
    if (allow_shared_memory(configured, kernel, DecodeRing<HD>::kBytes) != cudaSuccess) return static_cast<int>(cudaGetLastError());
    if (p.fresh_keys >= 0) {
        const cudaError_t launched = launch_overlapped(kernel, grid, dim3(kDecodeWarps * 32), DecodeRing<HD>::kBytes, stream, p);
        if (launched != cudaSuccess) return static_cast<int>(launched);
    } else {
        kernel<<<grid, kDecodeWarps * 32, DecodeRing<HD>::kBytes, stream>>>(p);
    }
    if (p.splits > 1)
        attention_decode_merge_kernel<HD><<<dim3(p.num_heads, tokens), HD >= 64 ? 64 : 32, 0, stream>>>(p.partial_out, p.partial_stats, out,
                                                                                                      p.token_list, p.num_heads, p.splits);
    return static_cast<int>(cudaGetLastError());
}

}  // namespace lb

extern "C" {

// How many CTAs of the kernel an SM holds at this head size (asked of the runtime for the current
// device: registers and the ring's shared memory decide); 0 if the head size is not supported.  The
// split plan counts rounds of resident CTAs with it.
int lb_attention_decode_ctas_per_sm(int head_dim) {
    int ctas = 0;
#define LB_DECODE_OCCUPANCY(HD)                                                                                          \
    case HD: {                                                                                                           \
        static lb::OncePerDevice configured;                                                                             \
        if (lb::allow_shared_memory(configured, lb::attention_decode_kernel<HD>, lb::DecodeRing<HD>::kBytes) != cudaSuccess) return 0; \
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas, lb::attention_decode_kernel<HD>, lb::kDecodeWarps * 32,  \
                                                          lb::DecodeRing<HD>::kBytes) != cudaSuccess) return 0;          \
        return ctas;                                                                                                     \
    }
    switch (head_dim) {
        LB_DECODE_OCCUPANCY(16) LB_DECODE_OCCUPANCY(32) LB_DECODE_OCCUPANCY(48) LB_DECODE_OCCUPANCY(64)
        LB_DECODE_OCCUPANCY(80) LB_DECODE_OCCUPANCY(96) LB_DECODE_OCCUPANCY(112) LB_DECODE_OCCUPANCY(128)
        default: return 0;
    }
#undef LB_DECODE_OCCUPANCY
}

// Floats of scratch the call needs: tokens * heads * splits * (head_dim + 2).  `tokens` counts the
// tokens that run: the length of `token_list`, or all tokens when it is null.
long long lb_attention_decode_scratch_floats(int tokens, int num_heads, int head_dim, int splits) {
    return static_cast<long long>(tokens) * num_heads * splits * (head_dim + 2);
}

// Returns 0, a CUDA error code, -1 for an unsupported type, or -2 for sizes the kernel does not take
// (head_dim must be a multiple of 16 up to 128, page_size a multiple of 16, the scale positive).
int lb_attention_decode(const void* q, const void* k_pages, const void* v_pages, void* out, float* scratch,
                        const int* positions, const int* token_segment, const int* block_table, const int* token_list,
                        int tokens, int num_heads, int num_groups, int head_dim, int page_size, int num_pages, int max_blocks,
                        float scale, int window, int splits, int blocks_per_split, int fresh_keys, int* status, cudaStream_t stream) {
    // fresh_keys >= 0: see DecodeParams (the caller's previous kernel on the stream writes at most that many of
    // the newest positions a token sees, and lets this kernel start early); -1: an ordinary launch.
    if (tokens == 0) return 0;
    if (page_size % 16 != 0 || num_heads % num_groups != 0 || splits < 1 || blocks_per_split < 1 || !(scale > 0.0f) || fresh_keys < -1) return -2;
    lb::DecodeParams p;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.k_pages = static_cast<const __nv_bfloat16*>(k_pages);
    p.v_pages = static_cast<const __nv_bfloat16*>(v_pages);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.partial_out = scratch;
    p.partial_stats = scratch + static_cast<size_t>(tokens) * num_heads * splits * head_dim;
    p.positions = positions;
    p.token_segment = token_segment;
    p.block_table = block_table;
    p.token_list = token_list;
    p.num_heads = num_heads;
    p.num_groups = num_groups;
    p.page_size = page_size;
    p.num_pages = num_pages;
    p.max_blocks = max_blocks;
    p.splits = splits;
    p.blocks_per_split = blocks_per_split;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = status;
    p.fresh_keys = fresh_keys;
    __nv_bfloat16* result = static_cast<__nv_bfloat16*>(out);
    switch (head_dim) {
        case 16: return lb::launch_decode<16>(p, result, tokens, stream);
        case 32: return lb::launch_decode<32>(p, result, tokens, stream);
        case 48: return lb::launch_decode<48>(p, result, tokens, stream);
        case 64: return lb::launch_decode<64>(p, result, tokens, stream);
        case 80: return lb::launch_decode<80>(p, result, tokens, stream);
        case 96: return lb::launch_decode<96>(p, result, tokens, stream);
        case 112: return lb::launch_decode<112>(p, result, tokens, stream);
        case 128: return lb::launch_decode<128>(p, result, tokens, stream);
        default: return -2;
    }
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// The same attention for callers that must not allocate (declared in attention_decode_static.h).
// It has no counterpart in the reference.
//
// lb_attention_decode needs scratch for the splits' partial results, which its caller allocates.
// Some callers cannot: code that runs while a stream is being captured into a CUDA graph under a
// memory pool it does not own, a host thread that must never enter the allocator's locks or a
// driver call that may synchronise, a plug-in living inside another program's memory budget.  For
// them the scratch is a fixed array in the library's own device image.  Every GPU that loads the
// library holds those 16 MiB until the process exits, whether or not the entry point is ever called.
// ---------------------------------------------------------------------------------------------
#include <mutex>
#include <cstdio>

namespace lb {

constexpr long long kStaticScratchFloats = 4ll << 20;   // 4,194,304 floats = 16 MiB: the stated maximum
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
static float* g_static_scratch_address[kMaxDevices] = {};   // per device, found at its first call
static std::mutex g_static_scratch_mutex;

static void describe(char* message, int capacity, const char* text, long long a = 0, long long b = 0) {
    if (message != nullptr && capacity > 0) snprintf(message, static_cast<size_t>(capacity), text, a, b);
}

}  // namespace lb

extern "C" int lb_attention_decode_static(const void* q, const void* k_pages, const void* v_pages, void* out, const int* positions,
                                          const int* token_segment, const int* block_table, const int* token_list, int tokens,
                                          int num_heads, int num_groups, int head_dim, int page_size, int num_pages, int max_blocks,
                                          float scale, int window, int splits, int blocks_per_split, int* status, cudaStream_t stream,
                                          char* error_message, int error_capacity) {
    if (tokens == 0) return 0;
    if (tokens < 0 || num_heads < 1 || splits < 1 || head_dim < 1) {
        lb::describe(error_message, error_capacity, "attention_decode_static: tokens, heads, splits and head_dim must be positive");
        return -2;
    }
    const long long needed = lb_attention_decode_scratch_floats(tokens, num_heads, head_dim, splits);
    if (needed > lb::kStaticScratchFloats) {
        lb::describe(error_message, error_capacity,
                     "attention_decode_static: tokens * heads * splits * (head_dim + 2) = %lld floats of scratch exceed the built-in %lld; "
                     "use fewer tokens or splits, or the allocating entry point",
                     needed, lb::kStaticScratchFloats);
        return -4;
    }
    int device = -1;
    cudaError_t error = cudaGetDevice(&device);
    if (error != cudaSuccess || device < 0 || device >= lb::kMaxDevices) {
        lb::describe(error_message, error_capacity, "attention_decode_static: no usable current device (cudaGetDevice gave %lld, device %lld)",
                     static_cast<long long>(error), device);
        return error != cudaSuccess ? static_cast<int>(error) : -2;
    }
    float* scratch = nullptr;
    {
        // In host code the array's name is only a stand-in for the symbol: its device address must be
        // asked for, once per device, with that device current (it is: it is the caller's).
        std::lock_guard<std::mutex> guard(lb::g_static_scratch_mutex);
        if (lb::g_static_scratch_address[device] == nullptr) {
            void* address = nullptr;
            error = cudaGetSymbolAddress(&address, lb::g_static_scratch);
            if (error != cudaSuccess || address == nullptr) {
                lb::describe(error_message, error_capacity, "attention_decode_static: cudaGetSymbolAddress failed with CUDA error %lld", static_cast<long long>(error));
                return error != cudaSuccess ? static_cast<int>(error) : -2;
            }
            lb::g_static_scratch_address[device] = static_cast<float*>(address);
        }
        scratch = lb::g_static_scratch_address[device];
    }
    // Every partial slot of this call is written by the first kernel before the second reads it, so
    // nothing left over from an earlier call needs clearing.
    const int code = lb_attention_decode(q, k_pages, v_pages, out, scratch, positions, token_segment, block_table, token_list, tokens, num_heads,
                                         num_groups, head_dim, page_size, num_pages, max_blocks, scale, window, splits, blocks_per_split, -1, status, stream);
    if (code == -2) lb::describe(error_message, error_capacity, "attention_decode_static: head_dim must be a multiple of 16 up to 128 and page_size a multiple of 16");
    else if (code != 0) lb::describe(error_message, error_capacity, "attention_decode_static: launch failed with CUDA error %lld", code);
    return code;
}
