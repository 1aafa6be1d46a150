// Paged attention for portions of prompts: tiles of 32 query tokens, tensor-core products, keys and
// values staged in shared memory and shared by the query heads of one K/V head.
//
// One CTA handles (tile of up to 32 consecutive tokens of one request, K/V head, chunk of up to 8 of
// its query heads); each warp owns one query head: two blocks of 16 rows (tokens) of S = Q K^T and of O = P V.
// Keys are visited in tiles of 64, copied asynchronously into shared memory (two buffers) from the
// request's pages; scores, softmax (base 2, online, one update per tile) and the output accumulate
// in 32-bit; P is rounded to bfloat16 for the second product.  Fragment layouts follow attention_decode.cu: channels
// are permuted so that a lane reads contiguous bytes of a key row, and keys are permuted inside a
// 16-key block so that a lane's probabilities meet contiguous bytes of the transposed value rows.
// Every tile starts at a key index that is a multiple of 64, whatever the portion's start, so the
// order of the sums for a token does not depend on how the prompt was cut.
#include "common.cuh"

namespace lb {

constexpr int kPrefillTile = 32;      // query tokens per CTA
constexpr int kPrefillKeys = 64;      // keys per shared-memory tile
constexpr int kPrefillMaxWarps = 8;   // query heads per CTA
constexpr float kPrefillMaxSlack = 8.0f;   // how far a row's maximum may outgrow its reference exponent (base 2)

__device__ __forceinline__ void mma_16816_prefill(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 2^x by the hardware's approximation (two units in the last place of float32); 2^-inf = 0.
__device__ __forceinline__ float exp2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16_prefill(float low, float high) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<const uint32_t*>(&pair);
}

__device__ __forceinline__ void prefill_copy_16(void* shared_destination, const void* global_source) {
    const uint32_t destination = static_cast<uint32_t>(__cvta_generic_to_shared(shared_destination));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(destination), "l"(global_source) : "memory");
}

struct PrefillParams {
    const __nv_bfloat16* q;         // [tokens, heads, hd]
    const __nv_bfloat16* k_pages;   // [pages, page_size, groups, hd]
    const __nv_bfloat16* v_pages;   // [pages, groups, hd, page_size]
    __nv_bfloat16* out;             // [tokens, heads, hd]
    const int* tiles;               // [num_tiles, 2]: first token, count
    const int* positions;
    const int* token_segment;
    const int* block_table;
    int num_heads, num_groups, page_size, num_pages, max_blocks;
    int window;
    float scale_log2;
    int* status;
};

// Shared-memory pitches (bytes) that keep the fragment reads free of bank conflicts.
template <int HD>
struct PrefillShared {
    static constexpr int kKeyPitch = HD * 2 + 16;                 // one key row
    static constexpr int kValuePitch = kPrefillKeys * 2 + 32;     // one channel row of 64 keys
    static constexpr int kKeyBytes = kPrefillKeys * kKeyPitch;
    static constexpr int kValueBytes = HD * kValuePitch;
    static constexpr int kStageBytes = kKeyBytes + kValueBytes;
};

// Where the 16-key blocks of a 64-key tile lie: lane b < 4 of every warp holds the page of block b
// (-1: outside [needed_first, needed_last] or without a page, to be filled with zeros) and the index
// of the block's first key inside that page.  One read of the block table per tile and warp,
// asked for a tile ahead of its use.
struct PrefillTileEntry {
    int page, offset;
};

__device__ __forceinline__ PrefillTileEntry prefill_lookup(const PrefillParams& p, int segment, int first, int needed_first, int needed_last, int lane,
                                                           bool& bad) {
    PrefillTileEntry entry{-1, 0};
    const int block_first = first + 16 * lane;
    if (lane < kPrefillKeys / 16 && block_first + 15 >= needed_first && block_first <= needed_last) {
        const int blocks_per_page = p.page_size / 16;
        const int block = block_first / 16, column = block / blocks_per_page;
        entry.offset = (block - column * blocks_per_page) * 16;
        entry.page = column < p.max_blocks ? p.block_table[static_cast<size_t>(segment) * p.max_blocks + column] : -1;
        if (entry.page < 0 || entry.page >= p.num_pages) {
            bad = true;
            entry.page = -1;
        }
    }
    return entry;
}

// Copies the 64 keys of a tile into stage memory from the pages that `entry` names; blocks without a
// page are zero-filled.  Every warp runs the loops the same number of times (the shuffles need it):
// the counts are multiples of 32 and so is the number of threads.
template <int HD>
__device__ __forceinline__ void prefill_load_tile(unsigned char* stage, const PrefillParams& p, int group, PrefillTileEntry entry) {
    using Shared = PrefillShared<HD>;
    constexpr int kChunksPerKey = HD / 8;   // 16-byte chunks in a key row
    unsigned char* keys = stage;
    unsigned char* values = stage + Shared::kKeyBytes;
    const int threads = blockDim.x;
    // keys: 64 rows of HD * 2 bytes
    for (int index = threadIdx.x; index < kPrefillKeys * kChunksPerKey; index += threads) {
        const int row = index / kChunksPerKey, chunk = index - row * kChunksPerKey;
        const int page = __shfl_sync(0xffffffffu, entry.page, row >> 4);
        const int in_page = __shfl_sync(0xffffffffu, entry.offset, row >> 4) + (row & 15);
        void* destination = keys + row * Shared::kKeyPitch + chunk * 16;
        if (page >= 0) {
            prefill_copy_16(destination, p.k_pages + ((static_cast<size_t>(page) * p.page_size + in_page) * p.num_groups + group) * HD + chunk * 8);
        } else {
            *reinterpret_cast<uint4*>(destination) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    // values: HD channel rows; each 16-key block contributes two 16-byte chunks per channel
    for (int index = threadIdx.x; index < HD * (kPrefillKeys / 8); index += threads) {
        const int channel = index / (kPrefillKeys / 8), chunk = index - channel * (kPrefillKeys / 8);   // chunk: 8 keys
        const int page = __shfl_sync(0xffffffffu, entry.page, chunk >> 1);
        const int in_page = __shfl_sync(0xffffffffu, entry.offset, chunk >> 1) + (chunk & 1) * 8;
        void* destination = values + channel * Shared::kValuePitch + chunk * 16;
        if (page >= 0) {
            prefill_copy_16(destination, p.v_pages + ((static_cast<size_t>(page) * p.num_groups + group) * HD + channel) * p.page_size + in_page);
        } else {
            *reinterpret_cast<uint4*>(destination) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
}

// grid (num_tiles, groups * head_chunks), blockDim = 32 * heads in the chunk (<= 8 warps).
// A tile has up to 16 * RB tokens; each warp owns RB blocks of 16 rows (tokens) of its head, which
// share every key and value fragment read from shared memory.
template <int HD, int RB>
__global__ void __launch_bounds__(kPrefillMaxWarps * 32)
attention_prefill_kernel(const PrefillParams p) {
    using Shared = PrefillShared<HD>;
    extern __shared__ __align__(16) unsigned char shared[];
    allow_next_kernel();   // the out-projection that follows may ask for its weights meanwhile
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int heads_per_group = p.num_heads / p.num_groups;
    const int head_chunks = (heads_per_group + kPrefillMaxWarps - 1) / kPrefillMaxWarps;
    const int group = blockIdx.y / head_chunks, head_chunk = blockIdx.y - group * head_chunks;
    const int head = group * heads_per_group + head_chunk * (blockDim.x >> 5) + warp;   // this warp's query head
    // A tile record holds up to kPrefillTile tokens; this CTA takes 16 * RB of them (grid.z covers the rest).
    // Tiles are listed in the order of the tokens; the last ones of a prompt see the most keys and start first.
    const int tile_record = gridDim.x - 1 - blockIdx.x;
    const int first_token = p.tiles[2 * tile_record] + 16 * RB * blockIdx.z;
    const int count = min(16 * RB, p.tiles[2 * tile_record + 1] - 16 * RB * static_cast<int>(blockIdx.z));
    if (count <= 0) return;
    const int segment = p.token_segment[first_token];
    const int first_position = p.positions[first_token], last_position = first_position + count - 1;
    const int first_visible = p.window > 0 ? max(0, first_position - p.window + 1) : 0;   // of the tile's first token
    const int tile_begin = (first_visible / kPrefillKeys) * kPrefillKeys;
    const int num_key_tiles = (last_position - tile_begin) / kPrefillKeys + 1;

    // Q fragments: rows g and g + 8 of row block rb are tokens first_token + 16 rb + g (+ 8); zero past the tile's end.
    uint32_t q_frag[RB][HD / 16][4];
#pragma unroll
    for (int rb = 0; rb < RB; ++rb) {
#pragma unroll
        for (int j = 0; j < HD / 16; ++j) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = 16 * rb + g + 8 * half;
                uint2 loaded = make_uint2(0u, 0u);
                if (row < count) {
                    const __nv_bfloat16* source = p.q + (static_cast<size_t>(first_token + row) * p.num_heads + head) * HD + t * (HD / 4) + 4 * j;
                    loaded = *reinterpret_cast<const uint2*>(source);
                }
                q_frag[rb][j][half] = loaded.x;
                q_frag[rb][j][2 + half] = loaded.y;
            }
        }
    }
    float out[RB][HD / 8][4];
    float row_max[RB][2], row_sum[RB][2];
    int row_position[RB][2], row_first[RB][2];
#pragma unroll
    for (int rb = 0; rb < RB; ++rb) {
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) out[rb][n][0] = out[rb][n][1] = out[rb][n][2] = out[rb][n][3] = 0.0f;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            row_max[rb][r] = -INFINITY;
            row_sum[rb][r] = 0.0f;
            row_position[rb][r] = first_position + 16 * rb + g + 8 * r;
            row_first[rb][r] = p.window > 0 ? max(0, row_position[rb][r] - p.window + 1) : 0;
        }
    }
    bool bad = false;

    prefill_load_tile<HD>(shared, p, group, prefill_lookup(p, segment, tile_begin, first_visible, last_position, lane, bad));
    PrefillTileEntry next_entry = prefill_lookup(p, segment, tile_begin + kPrefillKeys, first_visible, last_position, lane, bad);
    for (int tile = 0; tile < num_key_tiles; ++tile) {
        unsigned char* stage = shared + (tile & 1) * Shared::kStageBytes;
        const int key0 = tile_begin + tile * kPrefillKeys;
        if (tile + 1 < num_key_tiles) {
            prefill_load_tile<HD>(shared + ((tile + 1) & 1) * Shared::kStageBytes, p, group, next_entry);
            next_entry = prefill_lookup(p, segment, key0 + 2 * kPrefillKeys, first_visible, last_position, lane, bad);
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        unsigned char* values = stage + Shared::kKeyBytes;
        if (key0 + kPrefillKeys - 1 > last_position || key0 < first_visible) {
            // Keys past the tile's last token hold whatever was left in the page, and keys before the
            // first visible one are nobody's business: clear their values, since a zero probability
            // does not silence a non-finite value in the product.
            const int keep_from = first_visible - key0, keep_to = last_position - key0;   // keys [from, to] of this tile are real
            for (int index = threadIdx.x; index < HD * kPrefillKeys; index += blockDim.x) {
                const int channel = index / kPrefillKeys, key = index - channel * kPrefillKeys;
                if (key < keep_from || key > keep_to) *reinterpret_cast<__nv_bfloat16*>(values + channel * Shared::kValuePitch + key * 2) = __float2bfloat16_rn(0.0f);
            }
            __syncthreads();
        }
        // S = Q K^T for the whole tile: 16-key block `block`, half `b` of it -> s[.][2 * block + b].
        const int blocks_here = min(kPrefillKeys / 16, (last_position - key0) / 16 + 1);   // blocks with a key some token sees
        float s[RB][kPrefillKeys / 8][4];
#pragma unroll
        for (int block = 0; block < kPrefillKeys / 16; ++block) {
#pragma unroll
            for (int b = 0; b < 2; ++b) {
#pragma unroll
                for (int rb = 0; rb < RB; ++rb) s[rb][2 * block + b][0] = s[rb][2 * block + b][1] = s[rb][2 * block + b][2] = s[rb][2 * block + b][3] = 0.0f;
            }
            if (block < blocks_here) {
                // All fragments of the block first, then the products with the channel step outermost:
                // two products into the same accumulator are 2 * RB products apart.
                uint2 loaded[2][HD / 16];
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    const int key = block * 16 + 4 * (g >> 1) + 2 * b + (g & 1);
                    const unsigned char* row = stage + key * Shared::kKeyPitch + t * (HD / 4) * 2;
#pragma unroll
                    for (int j = 0; j < HD / 16; ++j) loaded[b][j] = *reinterpret_cast<const uint2*>(row + j * 8);
                }
#pragma unroll
                for (int j = 0; j < HD / 16; ++j) {
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
#pragma unroll
                        for (int rb = 0; rb < RB; ++rb) mma_16816_prefill(s[rb][2 * block + b], q_frag[rb][j], loaded[b][j].x, loaded[b][j].y);
                    }
                }
            }
        }
        // Softmax over the tile's 64 keys at once: one new maximum, one rescaling of the output.  Only
        // tiles that reach past some token's own position, or before some token's window, need masks.
        const bool needs_mask = key0 + kPrefillKeys - 1 > first_position || (p.window > 0 && key0 < last_position - p.window + 1);
        uint32_t p_frag[RB][kPrefillKeys / 16][4];
        float rescale[RB][2];
        if (needs_mask) {   // one branch for the whole tile: most tiles skip all of this
#pragma unroll
            for (int rb = 0; rb < RB; ++rb) {
#pragma unroll
                for (int n = 0; n < kPrefillKeys / 8; ++n) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int key = key0 + (n >> 1) * 16 + 4 * t + 2 * (n & 1) + (c & 1);
                        if (key < row_first[rb][c >> 1] || key > row_position[rb][c >> 1]) s[rb][n][c] = -INFINITY;
                    }
                }
            }
        }
#pragma unroll
        for (int rb = 0; rb < RB; ++rb) {
            float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < kPrefillKeys / 8; ++n) {
#pragma unroll
                for (int c = 0; c < 4; ++c) tile_max[c >> 1] = fmaxf(tile_max[c >> 1], s[rb][n][c]);
            }
            float shift[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
                tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
                // row_max is the exponent the row's terms are taken relative to, not its true maximum: it
                // follows the maximum only when that has grown by more than 8 (terms up to 2^8 lose
                // nothing in bfloat16 or in the 32-bit sums), so that the output is rarely rescaled.
                const float tile_top = tile_max[r] * p.scale_log2;   // the scale is positive
                const float new_max = tile_top > row_max[rb][r] + kPrefillMaxSlack ? tile_top : row_max[rb][r];
                shift[r] = new_max == -INFINITY ? 0.0f : new_max;   // a row that has seen no key yet: every term below is 2^-inf = 0
                rescale[rb][r] = exp2_fast(row_max[rb][r] - shift[r]);
                row_max[rb][r] = new_max;
            }
            float partial_sum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int n = 0; n < kPrefillKeys / 8; ++n) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int r = c >> 1;
                    s[rb][n][c] = exp2_fast(fmaf(s[rb][n][c], p.scale_log2, -shift[r]));
                    partial_sum[r] += s[rb][n][c];
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) row_sum[rb][r] = row_sum[rb][r] * rescale[rb][r] + partial_sum[r];
#pragma unroll
            for (int block = 0; block < kPrefillKeys / 16; ++block) {
                p_frag[rb][block][0] = pack_bf16_prefill(s[rb][2 * block][0], s[rb][2 * block][1]);
                p_frag[rb][block][1] = pack_bf16_prefill(s[rb][2 * block][2], s[rb][2 * block][3]);
                p_frag[rb][block][2] = pack_bf16_prefill(s[rb][2 * block + 1][0], s[rb][2 * block + 1][1]);
                p_frag[rb][block][3] = pack_bf16_prefill(s[rb][2 * block + 1][2], s[rb][2 * block + 1][3]);
            }
        }
        bool unchanged = true;
#pragma unroll
        for (int rb = 0; rb < RB; ++rb) unchanged = unchanged && rescale[rb][0] == 1.0f && rescale[rb][1] == 1.0f;
        if (!__all_sync(0xffffffffu, unchanged)) {
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) {
#pragma unroll
                for (int rb = 0; rb < RB; ++rb) {
                    out[rb][n][0] *= rescale[rb][0];
                    out[rb][n][1] *= rescale[rb][0];
                    out[rb][n][2] *= rescale[rb][1];
                    out[rb][n][3] *= rescale[rb][1];
                }
            }
        }
#pragma unroll
        for (int block = 0; block < kPrefillKeys / 16; ++block) {
            if (block < blocks_here) {
#pragma unroll
                for (int n = 0; n < HD / 8; ++n) {
                    const uint2 loaded = *reinterpret_cast<const uint2*>(values + (8 * n + g) * Shared::kValuePitch + (block * 16 + 4 * t) * 2);
#pragma unroll
                    for (int rb = 0; rb < RB; ++rb) mma_16816_prefill(out[rb][n], p_frag[rb][block], loaded.x, loaded.y);
                }
            }
        }
        __syncthreads();   // the stage is refilled two tiles later
    }
    if (bad) report_error(p.status, kBadPage);
#pragma unroll
    for (int rb = 0; rb < RB; ++rb) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            row_sum[rb][r] += __shfl_xor_sync(0xffffffffu, row_sum[rb][r], 1);
            row_sum[rb][r] += __shfl_xor_sync(0xffffffffu, row_sum[rb][r], 2);
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = 16 * rb + g + 8 * half;
            if (row >= count) continue;
            const float inverse = row_sum[rb][half] > 0.0f ? 1.0f / row_sum[rb][half] : 0.0f;
            __nv_bfloat16* destination = p.out + (static_cast<size_t>(first_token + row) * p.num_heads + head) * HD;
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) {
                *reinterpret_cast<uint32_t*>(destination + 8 * n + 2 * t) =
                    pack_bf16_prefill(out[rb][n][2 * half] * inverse, out[rb][n][2 * half + 1] * inverse);
            }
        }
    }
}

template <int HD>
int launch_prefill(const PrefillParams& p, int num_tiles, cudaStream_t stream) {
    using Shared = PrefillShared<HD>;
    const int heads_per_group = p.num_heads / p.num_groups;
    const int head_chunks = (heads_per_group + kPrefillMaxWarps - 1) / kPrefillMaxWarps;
    if (heads_per_group % head_chunks != 0) return -2;   // equal chunks only
    const int warps = heads_per_group / head_chunks;
    const int shared = 2 * Shared::kStageBytes;
    // Two row blocks per warp (tiles of 32 tokens) while the accumulators fit the registers.
    constexpr int row_blocks = HD <= 64 ? 2 : 1;
    auto kernel = attention_prefill_kernel<HD, row_blocks>;
    static OncePerDevice configured;
    if (allow_shared_memory(configured, kernel, shared) != cudaSuccess) return static_cast<int>(cudaGetLastError());
    kernel<<<dim3(num_tiles, p.num_groups * head_chunks, kPrefillTile / (16 * row_blocks)), warps * 32, shared, stream>>>(p);
    return static_cast<int>(cudaGetLastError());
}

}  // namespace lb

extern "C" {

// tiles: [num_tiles, 2] (first token, count <= 32), tokens of a tile consecutive in one request.
// Returns 0, a CUDA error, or -2 for sizes the kernel does not take (head_dim a multiple of 16 up
// to 128, page_size a multiple of 16, query heads per K/V head divisible into equal chunks of <= 8,
// a scale that is not positive).
int lb_attention_prefill(const void* q, const void* k_pages, const void* v_pages, void* out, const int* tiles, int num_tiles,
                         const int* positions, const int* token_segment, const int* block_table, int num_heads,
                         int num_groups, int head_dim, int page_size, int num_pages, int max_blocks, float scale, int window,
                         int* status, cudaStream_t stream) {
    if (num_tiles == 0) return 0;
    if (page_size % 16 != 0 || num_heads % num_groups != 0 || !(scale > 0.0f)) return -2;
    lb::PrefillParams p;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.k_pages = static_cast<const __nv_bfloat16*>(k_pages);
    p.v_pages = static_cast<const __nv_bfloat16*>(v_pages);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.tiles = tiles;
    p.positions = positions;
    p.token_segment = token_segment;
    p.block_table = block_table;
    p.num_heads = num_heads;
    p.num_groups = num_groups;
    p.page_size = page_size;
    p.num_pages = num_pages;
    p.max_blocks = max_blocks;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = status;
    switch (head_dim) {
        case 16: return lb::launch_prefill<16>(p, num_tiles, stream);
        case 32: return lb::launch_prefill<32>(p, num_tiles, stream);
        case 48: return lb::launch_prefill<48>(p, num_tiles, stream);
        case 64: return lb::launch_prefill<64>(p, num_tiles, stream);
        case 80: return lb::launch_prefill<80>(p, num_tiles, stream);
        case 96: return lb::launch_prefill<96>(p, num_tiles, stream);
        case 112: return lb::launch_prefill<112>(p, num_tiles, stream);
        case 128: return lb::launch_prefill<128>(p, num_tiles, stream);
        default: return -2;
    }
}

}  // extern "C"
