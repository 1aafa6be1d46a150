// Paged attention for portions of prompts on the fifth-generation tensor cores: scores and output
// live in tensor memory, keys, values and queries arrive by TMA.
//
// One CTA handles up to 128 rows = (consecutive tokens of one request) x (the query heads of one K/V
// head), which all see the same keys and values.  Keys are visited in tiles of 64, starting at a
// multiple of 64 whatever the portion's start.  Roles:
//   warp 0     one lane asks for Q once (a 3-D box: channels x the K/V head's query heads x tokens) and,
//              per tile and 16-key block, for a box of K rows (128-byte swizzle) and a box of the
//              transposed V page (32-byte swizzle), into two stages;
//   warp 1     allocates tensor memory; one lane issues  S = Q K^T  (M 128, N 64, four steps over the
//              64 channels) and, once the probabilities are in shared memory,  O += P V  (N 64
//              channels, four steps of 16 keys, one per V box);
//   warps 2-5  a thread per row: read the row's 64 scores from tensor memory, mask on edge tiles,
//              update the row's reference exponent and sum (32-bit, base 2, no shuffles: the row is
//              the thread's own), rescale the row of O in tensor memory when the exponent moved, write
//              P (bfloat16) into shared memory in the operand's swizzled layout; at the end divide the
//              row of O by its sum and store it.
// Several CTAs share an SM (64 KB of shared memory, 128 columns of tensor memory each), so that one's
// softmax runs under another's products.  Every wait is bounded and reports through the status word.
// Takes head size 64, pages that are multiples of 16 keys, up to 128 query heads per K/V head.
#include <type_traits>

#include "tcgen05.cuh"

namespace lb {

constexpr int kTaRows = 128;      // rows of a tile (lanes of tensor memory)
constexpr int kTaKeys = 64;       // keys per tile
constexpr int kTaHeadDim = 64;
constexpr int kTaThreads = 192;
constexpr int kTaTileTokens = 32;  // tokens of a tile record
constexpr float kTaMaxSlack = 8.0f;   // how far a row's maximum may outgrow its reference exponent (base 2)

struct TaParams {
    __nv_bfloat16* out;     // [tokens, heads, 64]
    const int* tiles;       // [num_tiles, 2]: first token, count <= 32
    const int* positions;
    const int* token_segment;
    const int* block_table;
    int num_heads, num_groups, tokens_per_cta;
    int page_size, num_pages, max_blocks, window;
    int page_shift;   // log2 of page_size if that is a power of two, else -1
    int split_tiles;  // > 0: the grid is pairs of CTAs (a cluster of two per tile record); a tile with at least this many key tiles is shared by its pair
    float scale_log2;
    int* status;
};

struct TaShared {
    static constexpr int kQBytes = kTaRows * kTaHeadDim * 2;           // 16 KB
    static constexpr int kPBytes = kTaRows * kTaKeys * 2;              // 16 KB
    static constexpr int kKeyBytes = kTaKeys * kTaHeadDim * 2;         // 8 KB: four boxes of 16 rows
    static constexpr int kValueBytes = kTaHeadDim * kTaKeys * 2;       // 8 KB: four boxes of 64 channels x 16 keys
    static constexpr int kStageBytes = kKeyBytes + kValueBytes;
    static constexpr int kBytes = kQBytes + kPBytes + 2 * kStageBytes + 1024 /* alignment */ + 256 /* barriers */;
};

__device__ __forceinline__ void tma_load_3d(void* destination, const CUtensorMap* map, int x, int y, int z, uint64_t* barrier) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_address(destination)), "l"(map), "r"(smem_address(barrier)), "r"(x), "r"(y), "r"(z)
        : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* destination, const CUtensorMap* map, int x, int y, int z, int w, uint64_t* barrier) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_address(destination)), "l"(map), "r"(smem_address(barrier)), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}

// Descriptor of a K-major tile with 32-byte swizzle: rows of 32 bytes (16 keys), groups of 8 rows 256 bytes apart.
__device__ __forceinline__ uint64_t value_box_descriptor(const void* tile) {
    const uint64_t address = smem_address(tile);
    return ((address & 0x3FFFFull) >> 4) | (1ull << 16) | (static_cast<uint64_t>(256 >> 4) << 32) | (1ull << 46) | (6ull << 61);
}

__device__ __forceinline__ void tmem_store_32(uint32_t address, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, "
        "%23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(address), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]),
          "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Two float32 values in one 64-bit register, for the packed arithmetic of sm_100 (one instruction for two
// fused multiply-adds or additions).
__device__ __forceinline__ uint64_t pack2(float low, float high) {
    uint64_t packed;
    asm("mov.b64 %0, {%1, %2};" : "=l"(packed) : "f"(low), "f"(high));
    return packed;
}
__device__ __forceinline__ void unpack2(uint64_t packed, float& low, float& high) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(low), "=f"(high) : "l"(packed));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__device__ __forceinline__ float exp2_hardware(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// grid (tiles, K/V heads, parts of a 32-token tile record), 192 threads.
template <bool PAIRED>
__global__ void __launch_bounds__(kTaThreads, 3)   // three CTAs per SM: one's softmax runs under the others' products
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                         const TaParams p) {
    extern __shared__ unsigned char raw_shared[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_shared) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* q_tile = base;
    unsigned char* p_tile = base + TaShared::kQBytes;
    unsigned char* stages = p_tile + TaShared::kPBytes;
    uint64_t* barriers = reinterpret_cast<uint64_t*>(stages + 2 * TaShared::kStageBytes);
    uint64_t* q_full = barriers;
    // Keys and values have barriers of their own: a stage's keys are free again as soon as S = Q K^T of
    // their tile is done, a whole softmax before its values are, and the keys of the tile after next
    // are then on their way that much earlier (with one barrier for both, the next tile's S waited
    // 0.7 us for its keys in every turn of the loop).
    uint64_t* k_full = barriers + 1;     // [2]
    uint64_t* k_free = barriers + 3;     // [2]
    uint64_t* v_full = barriers + 14;    // [2]
    uint64_t* v_free = barriers + 16;    // [2]
    uint64_t* s_ready = barriers + 5;
    uint64_t* p_ready = barriers + 6;
    uint64_t* pv_done = barriers + 7;
    uint64_t* s_free = barriers + 8;     // every softmax thread has read its row of scores for the last time
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(barriers + 9);
    __shared__ int failed;

    allow_next_kernel();   // the out-projection that follows may ask for its weights meanwhile
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_per_group = p.num_heads / p.num_groups;
    const int group = blockIdx.y;
    // Tiles are listed in the order of the tokens; the last ones of a prompt see the most keys and start first.
    // With split_tiles > 0 two CTAs (a cluster) stand behind every tile record: where the tile sees many keys,
    // each takes half of them and CTA 0 merges the halves at the end (CTA 1 sends its output, exponent and sum
    // into CTA 0's shared memory); where it sees few, CTA 1 leaves at once.  What bounds a launch of few tiles
    // is the chain of 64-key steps of its longest tile, and this halves it.
    constexpr bool paired = PAIRED;
    const int rank = paired ? static_cast<int>(cluster_rank()) : 0;
    const int records = paired ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
    const int record = records - 1 - (paired ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x));
    const int first_token = p.tiles[2 * record] + p.tokens_per_cta * blockIdx.z;
    const int count = min(p.tokens_per_cta, p.tiles[2 * record + 1] - p.tokens_per_cta * static_cast<int>(blockIdx.z));
    if (count <= 0) return;   // the whole CTA (and its partner): nothing has been set up yet
    const int segment = p.token_segment[first_token];
    const int first_position = p.positions[first_token], last_position = first_position + count - 1;
    const int first_visible = p.window > 0 ? max(0, first_position - p.window + 1) : 0;   // of the tile's first token
    int tile_begin = (first_visible / kTaKeys) * kTaKeys;
    int num_key_tiles = (last_position - tile_begin) / kTaKeys + 1;
    const bool shared_tile = paired && num_key_tiles >= p.split_tiles;
    if (paired && !shared_tile && rank == 1) return;   // CTA 0 does this tile alone and uses no cluster barrier
    if (shared_tile) {
        const int lower = num_key_tiles / 2;
        if (rank == 1) tile_begin += lower * kTaKeys;
        num_key_tiles = rank == 0 ? lower : num_key_tiles - lower;
    }

    if (threadIdx.x == 0) {
        barrier_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            barrier_init(&k_full[s], 1);
            barrier_init(&k_free[s], 1);
            barrier_init(&v_full[s], 1);
            barrier_init(&v_free[s], 1);
        }
        barrier_init(s_ready, 1);
        barrier_init(p_ready, 4);   // one arrival per softmax warp
        barrier_init(pv_done, 1);
        barrier_init(s_free, 4);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_address(tmem_slot)), "r"(128) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_scores = tmem_base, tmem_output = tmem_base + kTaKeys;

    if (warp == 0) {
        // Producer: the warp's first four lanes take one block of 16 keys each (its place in the block
        // table, its two boxes), so a tile costs the scheduler a quarter of the instructions one lane
        // would need; the other lanes idle along.
        if (lane == 0) {
            barrier_expect(q_full, static_cast<uint32_t>(p.tokens_per_cta * heads_per_group * kTaHeadDim * 2));
            tma_load_3d(q_tile, &map_q, 0, group * heads_per_group, first_token, q_full);
        }
        bool bad = false;
        // Blocks of 16 keys that some token of the tile sees and that have a page; the others are not
        // loaded (their scores are masked and their values cleared by the softmax warps).  A tile's entries
        // of the block table are read one tile ahead, so that the read's latency is not between a freed
        // stage and its next boxes.
        auto look_up = [&](int tile, int& page, int& offset) {
            page = -1;
            offset = 0;
            const int block_first = tile_begin + tile * kTaKeys + 16 * lane;
            if (lane < 4 && tile < num_key_tiles && block_first + 15 >= first_visible && block_first <= last_position) {
                const int column = p.page_shift >= 0 ? block_first >> p.page_shift : block_first / p.page_size;
                const int entry = column < p.max_blocks ? p.block_table[static_cast<size_t>(segment) * p.max_blocks + column] : -1;
                if (entry >= 0 && entry < p.num_pages) {
                    page = entry;
                    offset = block_first - column * p.page_size;
                } else {
                    bad = true;
                }
            }
        };
        int page, offset;
        look_up(0, page, offset);
        for (int tile = 0; tile < num_key_tiles; ++tile) {
            const int s = tile & 1;
            unsigned char* keys = stages + s * TaShared::kStageBytes;
            unsigned char* values = keys + TaShared::kKeyBytes;
            const int this_page = page, this_offset = offset;
            look_up(tile + 1, page, offset);
            const uint32_t bytes = 2048u * static_cast<uint32_t>(__popc(__ballot_sync(0xffffffffu, this_page >= 0)));
            if (tile >= 2 && !__all_sync(0xffffffffu, barrier_wait_parked(&k_free[s], ((tile >> 1) - 1) & 1))) {
                atomicExch(&failed, 1);
                break;
            }
            if (lane == 0) barrier_expect(&k_full[s], bytes);
            if (this_page >= 0) tma_load_4d(keys + lane * 2048, &map_k, 0, group, this_offset, this_page, &k_full[s]);
            if (tile >= 2 && !__all_sync(0xffffffffu, barrier_wait_parked(&v_free[s], ((tile >> 1) - 1) & 1))) {
                atomicExch(&failed, 1);
                break;
            }
            if (lane == 0) barrier_expect(&v_full[s], bytes);
            if (this_page >= 0) tma_load_4d(values + lane * 2048, &map_v, this_offset, 0, group, this_page, &v_full[s]);
        }
        if (__any_sync(0xffffffffu, bad) && lane == 0) report_error(p.status, kBadPage);
    } else if (warp == 1 && lane == 0) {
        // Product issuer.  It waits parked: three CTAs' issuers polling on one scheduler took the ALU
        // slots of the softmax warps there, and every tile waits for its slowest softmax warp.
        constexpr uint32_t idesc = instruction_descriptor<kTaKeys>();   // N = 64 for both products (64 keys, 64 channels)
        bool ok = barrier_wait(q_full, 0);
        if (!ok) atomicExch(&failed, 1);
        const uint64_t desc_q = tile_descriptor(q_tile), desc_p = tile_descriptor(p_tile);
        // S = Q K^T of tile t + 1 is issued as soon as the softmax threads have read S of tile t for the
        // last time, before their P is complete: it runs under the rest of their work, and the scores of
        // the next tile are there when they come for them.
        auto issue_scores = [&](int tile) {
            if (!barrier_wait_parked(&k_full[tile & 1], (tile >> 1) & 1)) return false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t desc_k = tile_descriptor(stages + (tile & 1) * TaShared::kStageBytes);
#pragma unroll
            for (int k = 0; k < kTaHeadDim / 16; ++k) mma_f16(tmem_scores, desc_q + 2 * k, desc_k + 2 * k, idesc, k > 0);
            mma_commit(s_ready);
            mma_commit(&k_free[tile & 1]);
            return true;
        };
        if (ok && !issue_scores(0)) {
            atomicExch(&failed, 1);
            ok = false;
        }
        for (int tile = 0; tile < num_key_tiles && ok; ++tile) {
            const int s = tile & 1;
            unsigned char* values = stages + s * TaShared::kStageBytes + TaShared::kKeyBytes;
            if (tile + 1 < num_key_tiles) {
                if (!barrier_wait_parked(s_free, tile & 1)) {
                    atomicExch(&failed, 1);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (!issue_scores(tile + 1)) {
                    atomicExch(&failed, 1);
                    break;
                }
            }
            if (!barrier_wait_parked(p_ready, tile & 1) || !barrier_wait_parked(&v_full[s], (tile >> 1) & 1)) {
                atomicExch(&failed, 1);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int k = 0; k < kTaKeys / 16; ++k) mma_f16(tmem_output, desc_p + 2 * k, value_box_descriptor(values + k * 2048), idesc, tile > 0 || k > 0);
            mma_commit(&v_free[s]);
            mma_commit(pv_done);
        }
    } else if (warp >= 2) {
        // A thread per row.  Row r is token r / heads_per_group of the CTA's tokens, query head r % heads_per_group.
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const int token_local = row / heads_per_group, head_local = row - token_local * heads_per_group;
        const bool valid_row = token_local < count;
        const int row_position = first_position + token_local;
        const int row_first = p.window > 0 ? max(0, row_position - p.window + 1) : 0;
        const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
        float reference = -INFINITY, row_sum = 0.0f;
        bool ok = true;
        // The warp's lanes leave the loop together or not at all: what follows a wait is warp-wide.
        // One lane waits, parked in hardware: with three CTAs on an SM a warp waits for nearly half of
        // the time, and polling warps took the ALU slots that the other CTAs' softmax needed.
        auto wait_together = [](uint64_t* barrier, uint32_t parity) {
            // every lane waits on the same barrier (one instruction per warp, as for one lane; no exchange after it)
            return __all_sync(0xffffffffu, barrier_wait_parked(barrier, parity));
        };
        for (int tile = 0; tile < num_key_tiles; ++tile) {
            const int s = tile & 1;
            const int key0 = tile_begin + tile * kTaKeys;
            if (!wait_together(s_ready, tile & 1)) {
                ok = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // Only tiles that reach past some token's own position, or before some token's window, need masks.
            const bool needs_mask = key0 + kTaKeys - 1 > first_position || (p.window > 0 && key0 < last_position - p.window + 1);
            // The row is read twice, 32 scores at a time (once for its maximum, once for its terms): a
            // thread then needs half the registers, and three CTAs fit an SM.  Both passes exist with and
            // without the mask, chosen by one branch per tile: with the test inside the loops the
            // compiler evaluated the mask's comparisons for every score of every tile (four ALU
            // instructions per score and pass, which made the ALU pipe the kernel's limit).
            float tops[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            auto row_maximum = [&](auto masked) {
                constexpr bool kMasked = decltype(masked)::value;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t raw[32];
                    tmem_load_32(tmem_scores + lane_field + 32 * half, raw);
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float pair[2];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            pair[e] = __uint_as_float(raw[i + e]);
                            if constexpr (kMasked) {
                                const int key = key0 + 32 * half + i + e;
                                if (key < row_first || key > row_position) pair[e] = -INFINITY;
                            }
                        }
                        tops[(i >> 1) & 3] = max3(tops[(i >> 1) & 3], pair[0], pair[1]);   // one instruction for two scores
                    }
                }
            };
            if (needs_mask) row_maximum(std::true_type{});
            else row_maximum(std::false_type{});
            float top = fmaxf(fmaxf(tops[0], tops[1]), fmaxf(tops[2], tops[3]));
            // `reference` is the exponent the row's terms are taken relative to; it follows the row's maximum
            // only when that has grown by more than 2^8, so that the output is rarely rescaled.
            top *= p.scale_log2;   // the scale is positive
            const float moved = top > reference + kTaMaxSlack ? top : reference;
            const float shift = moved == -INFINITY ? 0.0f : moved;   // a row that has seen no key yet: every term below is 2^-inf = 0
            const float rescale = exp2_hardware(reference - shift);
            reference = moved;
            if (tile > 0) {
                // The products of the tile before have finished: P may be overwritten and O rescaled.
                if (!wait_together(pv_done, (tile - 1) & 1)) {
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (__any_sync(0xffffffffu, rescale != 1.0f)) {
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        uint32_t held[32];
                        tmem_load_32(tmem_output + lane_field + 32 * half, held);
#pragma unroll
                        for (int i = 0; i < 32; ++i) held[i] = __float_as_uint(__uint_as_float(held[i]) * rescale);
                        tmem_store_32(tmem_output + lane_field + 32 * half, held);
                    }
                }
            }
            float partials[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            uint64_t sums2[4] = {0ull, 0ull, 0ull, 0ull};   // pairs of 0.0f
            const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), shift2 = pack2(-shift, -shift);
            const uint32_t p_row = smem_address(p_tile) + static_cast<uint32_t>(row) * 128u;   // a 32-bit shared-memory address: plain shared stores
            auto row_terms = [&](auto masked) {
                constexpr bool kMasked = decltype(masked)::value;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t raw[32];
                    tmem_load_32(tmem_scores + lane_field + 32 * half, raw);
                    if (half == 1) {
                        // the row's scores are in registers: the next tile's may overwrite them
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) barrier_arrive(s_free);
                    }
#pragma unroll
                    for (int chunk = 0; chunk < 4; ++chunk) {
                        uint4 packed;
                        __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            float terms[2];
                            if constexpr (kMasked) {
#pragma unroll
                                for (int e = 0; e < 2; ++e) {
                                    const int index = 8 * chunk + 2 * i + e;
                                    float score = __uint_as_float(raw[index]);
                                    const int key = key0 + 32 * half + index;
                                    if (key < row_first || key > row_position) score = -INFINITY;
                                    terms[e] = exp2_hardware(fmaf(score, p.scale_log2, -shift));
                                }
                                partials[i] += terms[0] + terms[1];
                            } else {
                                // two scores per instruction: the scaled difference, and the running sums
                                const int index = 8 * chunk + 2 * i;
                                float low, high;
                                unpack2(fma2(pack2(__uint_as_float(raw[index]), __uint_as_float(raw[index + 1])), scale2, shift2), low, high);
                                terms[0] = exp2_hardware(low);
                                terms[1] = exp2_hardware(high);
                                sums2[i] = add2(sums2[i], pack2(terms[0], terms[1]));
                            }
                            pairs[i] = __floats2bfloat162_rn(terms[0], terms[1]);
                        }
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"   // the operand's 128-byte swizzle
                                     ::"r"(p_row + static_cast<uint32_t>(((4 * half + chunk) ^ (row & 7)) << 4)), "r"(packed.x), "r"(packed.y), "r"(packed.z), "r"(packed.w)
                                     : "memory");
                    }
                }
            };
            if (needs_mask) row_terms(std::true_type{});
            else row_terms(std::false_type{});
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float low, high;
                unpack2(sums2[i], low, high);
                partials[i] += low + high;
            }
            const float partial = (partials[0] + partials[1]) + (partials[2] + partials[3]);
            row_sum = row_sum * rescale + partial;
            if (needs_mask) {
                // Keys outside [first visible, last position] of the tile hold whatever was left in the page,
                // or were not loaded at all: clear their values, since a zero probability does not silence
                // a non-finite value in the product.  64 channels x 64 keys, two threads per channel.
                if (!wait_together(&v_full[s], (tile >> 1) & 1)) {
                    ok = false;
                    break;
                }
                unsigned char* values = stages + s * TaShared::kStageBytes + TaShared::kKeyBytes;
                const int channel = row & 63, key_half = row >> 6;
                for (int i = 0; i < 32; ++i) {
                    const int local_key = 32 * key_half + i, key = key0 + local_key;
                    if (key < first_visible || key > last_position) {
                        const int block = local_key >> 4, in_block = local_key & 15;
                        // 32-byte swizzle: the 16-byte half of a 32-byte row is flipped in rows 4-7 of every 8
                        unsigned char* address = values + block * 2048 + channel * 32 + ((((in_block >> 3) ^ (channel >> 2)) & 1) << 4) + (in_block & 7) * 2;
                        *reinterpret_cast<__nv_bfloat16*>(address) = __float2bfloat16_rn(0.0f);
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P and the cleared values, seen by the products
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();   // every lane's P, fenced, before the warp's one arrival
            if (lane == 0) barrier_arrive(p_ready);
        }
        if (ok && !wait_together(pv_done, (num_key_tiles - 1) & 1)) ok = false;
        if (!ok) atomicExch(&failed, 1);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // A tile shared by two CTAs: when both have been through their keys (first cluster barrier: CTA 0's
        // shared memory is free), CTA 1 sends its unnormalised output row, exponent and sum there; after the
        // second barrier CTA 0 merges.  The other warps of both CTAs meet the same barriers below.
        float* const received = reinterpret_cast<float*>(base);                  // [128 rows][64] over the Q and P tiles
        float* const received_scalars = reinterpret_cast<float*>(stages);        // [128 rows][2]
        if (shared_tile) cluster_sync();
        if (shared_tile && rank == 1) {
            const uint32_t remote_row = cluster_address(received + row * kTaHeadDim, 0);
            const uint32_t remote_scalars = cluster_address(received_scalars + row * 2, 0);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t held[32];
                tmem_load_32(tmem_output + lane_field + 32 * half, held);
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(remote_row + static_cast<uint32_t>((32 * half + i) * 4)), "r"(held[i]),
                                 "r"(held[i + 1]), "r"(held[i + 2]), "r"(held[i + 3])
                                 : "memory");
            }
            asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(remote_scalars), "f"(reference), "f"(row_sum) : "memory");
        }
        if (shared_tile) cluster_sync();
        if (rank == 0) {
            float mine = 1.0f, theirs = 0.0f;   // weights of the two halves
            if (shared_tile) {
                const float other_reference = received_scalars[row * 2], other_sum = received_scalars[row * 2 + 1];
                const float top = fmaxf(reference, other_reference);
                mine = top == -INFINITY ? 0.0f : exp2_hardware(reference - top);
                theirs = top == -INFINITY ? 0.0f : exp2_hardware(other_reference - top);
                row_sum = row_sum * mine + other_sum * theirs;
            }
            const float inverse = row_sum > 0.0f ? 1.0f / row_sum : 0.0f;
            __nv_bfloat16* destination = p.out + (static_cast<size_t>(first_token + token_local) * p.num_heads + group * heads_per_group + head_local) * kTaHeadDim;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t held[32];
                tmem_load_32(tmem_output + lane_field + 32 * half, held);
                if (valid_row && ok) {
#pragma unroll
                    for (int chunk = 0; chunk < 4; ++chunk) {
                        float values[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) values[i] = __uint_as_float(held[8 * chunk + i]) * mine;
                        if (shared_tile) {
                            const float4 low = *reinterpret_cast<const float4*>(received + row * kTaHeadDim + 32 * half + 8 * chunk);
                            const float4 high = *reinterpret_cast<const float4*>(received + row * kTaHeadDim + 32 * half + 8 * chunk + 4);
                            values[0] += low.x * theirs, values[1] += low.y * theirs, values[2] += low.z * theirs, values[3] += low.w * theirs;
                            values[4] += high.x * theirs, values[5] += high.y * theirs, values[6] += high.z * theirs, values[7] += high.w * theirs;
                        }
                        uint4 packed;
                        __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                        for (int i = 0; i < 4; ++i) pairs[i] = __floats2bfloat162_rn(values[2 * i] * inverse, values[2 * i + 1] * inverse);
                        *reinterpret_cast<uint4*>(destination + 32 * half + 8 * chunk) = packed;
                    }
                }
            }
        }
    }
    if (shared_tile && warp < 2) {
        // loader and issuer: the two cluster barriers of the softmax warps above
        cluster_sync();
        cluster_sync();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (failed) {
        // Let whatever copies are still in flight land before the shared memory goes away.
        if (threadIdx.x == 0) report_error(p.status, kWaitTimeout);
        for (int spin = 0; spin < 2000; ++spin) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(128) : "memory");
    }
}

// A tensor map of bfloat16 elements with up to four dimensions (innermost first).
static bool make_paged_map(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes, const cuuint32_t* box,
                           CUtensorMapSwizzle swizzle) {
    EncodeTiled encode = encode_tiled();
    if (encode == nullptr) return false;
    const cuuint32_t element_strides[4] = {1, 1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base), dims, strides_bytes, box, element_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace lb

extern "C" {

// Same arguments as lb_attention_prefill plus the number of tokens in q.  Returns 0, a CUDA error, -2 for
// sizes the kernel does not take (head_dim other than 64, page_size no multiple of 16, more than 128 query
// heads per K/V head, a scale that is not positive, pointers not 16-byte aligned), -5 if no tensor map
// could be made.
int lb_attention_prefill_tcgen05(const void* q, const void* k_pages, const void* v_pages, void* out, const int* tiles, int num_tiles, int tokens,
                                 const int* positions, const int* token_segment, const int* block_table, int num_heads, int num_groups,
                                 int head_dim, int page_size, int num_pages, int max_blocks, float scale, int window, int split_tiles, int* status,
                                 cudaStream_t stream) {
    // split_tiles > 0: a pair of CTAs per tile record; a tile that sees at least that many tiles of 64 keys is
    // shared by its pair (for launches of few tiles, which the longest tile's chain of keys bounds).
    if (num_tiles == 0 || tokens == 0) return 0;
    if (split_tiles < 0 || split_tiles == 1) return -2;
    if (head_dim != lb::kTaHeadDim || page_size % 16 != 0 || num_groups < 1 || num_heads % num_groups != 0 || num_heads / num_groups > lb::kTaRows ||
        !(scale > 0.0f))
        return -2;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_pages) | reinterpret_cast<uintptr_t>(v_pages) | reinterpret_cast<uintptr_t>(out)) & 15)
        return -2;
    const int heads_per_group = num_heads / num_groups;
    lb::TaParams p;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.tiles = tiles;
    p.positions = positions;
    p.token_segment = token_segment;
    p.block_table = block_table;
    p.num_heads = num_heads;
    p.num_groups = num_groups;
    p.tokens_per_cta = lb::kTaRows / heads_per_group < lb::kTaTileTokens ? lb::kTaRows / heads_per_group : lb::kTaTileTokens;
    p.page_size = page_size;
    p.page_shift = -1;
    for (int shift = 0; shift < 31; ++shift)
        if ((1 << shift) == page_size) p.page_shift = shift;
    p.num_pages = num_pages;
    p.max_blocks = max_blocks;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = status;

    CUtensorMap map_q, map_k, map_v;
    {
        const cuuint64_t dims[3] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(num_heads), static_cast<cuuint64_t>(tokens)};
        const cuuint64_t strides[2] = {static_cast<cuuint64_t>(head_dim) * 2, static_cast<cuuint64_t>(num_heads) * head_dim * 2};
        const cuuint32_t box[3] = {static_cast<cuuint32_t>(head_dim), static_cast<cuuint32_t>(heads_per_group), static_cast<cuuint32_t>(p.tokens_per_cta)};
        if (!lb::make_paged_map(&map_q, q, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -5;
    }
    {
        const cuuint64_t dims[4] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(num_groups), static_cast<cuuint64_t>(page_size),
                                    static_cast<cuuint64_t>(num_pages)};
        const cuuint64_t strides[3] = {static_cast<cuuint64_t>(head_dim) * 2, static_cast<cuuint64_t>(num_groups) * head_dim * 2,
                                       static_cast<cuuint64_t>(page_size) * num_groups * head_dim * 2};
        const cuuint32_t box[4] = {static_cast<cuuint32_t>(head_dim), 1, 16, 1};
        if (!lb::make_paged_map(&map_k, k_pages, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -5;
    }
    {
        const cuuint64_t dims[4] = {static_cast<cuuint64_t>(page_size), static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(num_groups),
                                    static_cast<cuuint64_t>(num_pages)};
        const cuuint64_t strides[3] = {static_cast<cuuint64_t>(page_size) * 2, static_cast<cuuint64_t>(head_dim) * page_size * 2,
                                       static_cast<cuuint64_t>(num_groups) * head_dim * page_size * 2};
        const cuuint32_t box[4] = {16, static_cast<cuuint32_t>(head_dim), 1, 1};
        if (!lb::make_paged_map(&map_v, v_pages, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_32B)) return -5;
    }
    static lb::OncePerDevice configured, configured_paired;
    if (lb::allow_shared_memory(configured, lb::attention_tcgen05_kernel<false>, lb::TaShared::kBytes) != cudaSuccess) return static_cast<int>(cudaGetLastError());
    if (split_tiles > 0 && lb::allow_shared_memory(configured_paired, lb::attention_tcgen05_kernel<true>, lb::TaShared::kBytes) != cudaSuccess)
        return static_cast<int>(cudaGetLastError());
    p.split_tiles = split_tiles;
    const unsigned parts = static_cast<unsigned>((lb::kTaTileTokens + p.tokens_per_cta - 1) / p.tokens_per_cta);
    if (split_tiles == 0) {
        const dim3 grid(num_tiles, num_groups, parts);
        lb::attention_tcgen05_kernel<false><<<grid, lb::kTaThreads, lb::TaShared::kBytes, stream>>>(map_q, map_k, map_v, p);
        return static_cast<int>(cudaGetLastError());
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * num_tiles, num_groups, parts);
    config.blockDim = dim3(lb::kTaThreads);
    config.dynamicSmemBytes = lb::TaShared::kBytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = 2;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    const cudaError_t launched = cudaLaunchKernelEx(&config, lb::attention_tcgen05_kernel<true>, map_q, map_k, map_v, p);
    if (launched != cudaSuccess) return static_cast<int>(launched);
    return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
