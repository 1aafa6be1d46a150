// Matrix products on the fifth-generation tensor cores (tcgen05) for steps of more than 16 tokens:
//     Y[token, n] = sum_k X[token, k] * W[n, k]      X: [tokens, K] bfloat16, W: [N, K] bfloat16
// computed "swapped", D = W X^T, so that rows of W fill the 128 lanes of the accumulator whatever
// the number of tokens, which become its columns (32 to 128 per CTA).
//
// One CTA owns a 128 x BN tile of D and a slice of K.  Its warps have fixed roles:
//   warp 0     one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of the W and X
//              tiles of each 64-column block into a ring of shared-memory stages;
//   warp 1     allocates tensor memory, and one lane issues tcgen05.mma (M 128, N BN, K 16) four
//              times per stage, committing each stage back to the producer and, after the last
//              block, the accumulator to the epilogue;
//   warps 2-5  read the accumulator from tensor memory (tcgen05.ld, one lane quarter each, a lane
//              per row of W) and store it: bfloat16, float32, added to the 32-bit residual stream,
//              or as a 32-bit partial of a K slice.
// K slices (grid.z) are for steps with few tokens, where 128-row tiles alone leave most SMs idle;
// their partials are summed in slice order by a second kernel, so results do not depend on timing.
// Every wait on a barrier is bounded: on expiry the CTA records kWaitTimeout, lets copies in flight
// land, frees its tensor memory and returns.
#include "tcgen05.cuh"

namespace lb {

constexpr int kTcRows = 128;         // rows of W per CTA (the accumulator's lanes)
constexpr int kTcBlockK = 64;        // columns per stage: 128 bytes of bfloat16, one swizzle atom
constexpr int kTcThreads = 192;

enum TcEpilogue : int { kTcStore = 0, kTcStoreFloat = 1, kTcResidualAdd = 2, kTcPartial = 3, kTcGated = 4 };

struct TcParams {
    void* out;          // [tokens, n] bfloat16 / float32 / residual, or partials [slices, tokens, n]
    int tokens, n, k;
    int blocks_per_slice;   // 64-column blocks of K per slice
    int epilogue;
    int hidden;         // kTcGated: W is [2 * hidden, k], rows [up ; gate]; out is [tokens, hidden]
    int activation;
    int bulk_store;     // the walking kernel writes its output by bulk tensor stores (rows of the output 16-byte aligned)
    int early_successor;   // the one-tile kernel lets the kernel after it start before it has finished
    int* status;
};

template <int BN, int STAGES>
struct TcShared {
    static constexpr int kWBytes = kTcRows * kTcBlockK * 2;
    static constexpr int kXBytes = BN * kTcBlockK * 2;
    static constexpr int kStageBytes = kWBytes + kXBytes;
    static constexpr int kTurnedBytes = BN * (kTcRows + 4) * 4;   // the epilogue's turned tile, float32 worst case
    static constexpr int kTileBytes = STAGES * kStageBytes > kTurnedBytes ? STAGES * kStageBytes : kTurnedBytes;
    static constexpr int kBytes = kTileBytes + 1024 /* alignment slack */ + 256 /* barriers */;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kTcThreads)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const TcParams p) {
    using Shared = TcShared<BN, STAGES>;
    constexpr int kColumns = BN < 32 ? 32 : BN;   // tensor-memory columns: a power of two, at least 32
    extern __shared__ unsigned char raw_shared[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_shared) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* barriers = reinterpret_cast<uint64_t*>(tiles + Shared::kTileBytes);
    uint64_t* full = barriers;                 // [STAGES] a stage's tiles have landed
    uint64_t* empty = barriers + STAGES;       // [STAGES] a stage's products are done
    uint64_t* accumulated = barriers + 2 * STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(barriers + 2 * STAGES + 1);
    __shared__ int failed;

    // With more than 16 tokens the successor may start early (measured: 1.6 % of a 64-token decode step, 2.7 %
    // of a 64-token prompt).  With fewer it is a weight-streaming product that pulls its weights towards L2
    // while this kernel's tiles of W stream in, which cost more than its early start gained (1.05 against
    // 0.97 ms a step).
    if (p.early_successor) allow_next_kernel();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Gated: 64 "up" rows and the 64 "gate" rows that belong to them share the CTA.
    const bool gated = p.epilogue == kTcGated;
    const int row0 = blockIdx.x * (gated ? kTcRows / 2 : kTcRows), token0 = blockIdx.y * BN;
    const int total_blocks = (p.k + kTcBlockK - 1) / kTcBlockK;
    const int first_block = blockIdx.z * p.blocks_per_slice;
    const int num_blocks = min(p.blocks_per_slice, total_blocks - first_block);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            barrier_init(&full[s], 1);
            barrier_init(&empty[s], 1);
        }
        barrier_init(accumulated, 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_address(tmem_slot)), "r"(kColumns) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // Producer.  The weights do not depend on the kernel before this one: the first round of
        // stages asks for its tiles of W at once, and only the tiles of X wait for that kernel.
        const int first_round = min(STAGES, num_blocks);
        for (int block = 0; block < first_round; ++block) {
            unsigned char* stage = tiles + block * Shared::kStageBytes;
            barrier_expect(&full[block], Shared::kStageBytes);
            const int column = (first_block + block) * kTcBlockK;
            tma_load_2d(stage, &map_w, column, row0, &full[block]);
            if (gated) tma_load_2d(stage + Shared::kWBytes / 2, &map_w, column, p.hidden + row0, &full[block]);
        }
        wait_for_previous_kernel();
        for (int block = 0; block < first_round; ++block)
            tma_load_2d(tiles + block * Shared::kStageBytes + Shared::kWBytes, &map_x, (first_block + block) * kTcBlockK, token0, &full[block]);
        for (int block = first_round; block < num_blocks; ++block) {
            const int s = block % STAGES, round = block / STAGES;
            if (!barrier_wait(&empty[s], (round - 1) & 1)) {
                atomicExch(&failed, 1);
                break;
            }
            unsigned char* stage = tiles + s * Shared::kStageBytes;
            barrier_expect(&full[s], Shared::kStageBytes);
            const int column = (first_block + block) * kTcBlockK;
            tma_load_2d(stage, &map_w, column, row0, &full[s]);
            if (gated) tma_load_2d(stage + Shared::kWBytes / 2, &map_w, column, p.hidden + row0, &full[s]);
            tma_load_2d(stage + Shared::kWBytes, &map_x, column, token0, &full[s]);
        }
    } else if (warp == 1 && lane == 0) {
        // Product issuer.
        constexpr uint32_t idesc = instruction_descriptor<BN>();
        bool ok = true;
        for (int block = 0; block < num_blocks && ok; ++block) {
            const int s = block % STAGES, round = block / STAGES;
            if (!barrier_wait(&full[s], round & 1)) {
                atomicExch(&failed, 1);
                ok = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            unsigned char* stage = tiles + s * Shared::kStageBytes;
            const uint64_t desc_w = tile_descriptor(stage), desc_x = tile_descriptor(stage + Shared::kWBytes);
#pragma unroll
            for (int k = 0; k < kTcBlockK / 16; ++k) {
                // 16 columns further along K = 32 bytes inside the swizzle atom = 2 in descriptor units
                mma_f16(tmem_base, desc_w + 2 * k, desc_x + 2 * k, idesc, block > 0 || k > 0);
            }
            mma_commit(&empty[s]);
        }
        if (ok) mma_commit(accumulated);
    } else if (warp >= 2) {
        // Epilogue: warp w may touch lanes 32 * (w % 4) ... + 31 of tensor memory.  The accumulator holds
        // a row of W per lane and a token per column, the output wants a token's rows side by side, so
        // the tile is turned over in shared memory (the stages are free once the accumulator is
        // complete) and leaves in 16-byte pieces.
        const int quarter = warp & 3;
        const int local_row = quarter * 32 + lane;
        const int epilogue_thread = threadIdx.x - 64;   // 0..127
        wait_for_previous_kernel();   // before anything of the output is read or written
        bool ok = num_blocks > 0 ? barrier_wait(accumulated, 0) : true;
        if (!ok) atomicExch(&failed, 1);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const bool as_bfloat16 = p.epilogue == kTcStore || gated;
        // Turned tile: [BN tokens][128 rows] of bfloat16 or float32, rows padded against bank conflicts.
        constexpr int kPitchHalf = kTcRows + 8, kPitchFloat = kTcRows + 4;
        if (ok) {
#pragma unroll 1
            for (int column = 0; column < BN; column += 16) {
                uint32_t v[16];
                if (num_blocks > 0) {
                    const uint32_t address = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(column);
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                        : "r"(address)
                        : "memory");
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = 0u;
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if (as_bfloat16) reinterpret_cast<__nv_bfloat16*>(tiles)[(column + i) * kPitchHalf + local_row] = __float2bfloat16_rn(__uint_as_float(v[i]));
                    else reinterpret_cast<float*>(tiles)[(column + i) * kPitchFloat + local_row] = __uint_as_float(v[i]);
                }
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps
        if (ok) {
            const bool vector_ok = p.n % 8 == 0 && row0 + kTcRows <= p.n;
            if (gated) {
                // 8 pieces of 8 outputs per token: up rows 0..63 of the turned tile, their gates 64 rows further
                for (int piece = epilogue_thread; piece < BN * 8; piece += 128) {
                    const int token_local = piece >> 3, part = piece & 7;
                    const int token = token0 + token_local;
                    if (token >= p.tokens) continue;
                    const __nv_bfloat16* up = reinterpret_cast<const __nv_bfloat16*>(tiles) + token_local * kPitchHalf + part * 8;
                    const __nv_bfloat16* gate = up + kTcRows / 2;
                    __nv_bfloat16 result[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float g = __bfloat162float(gate[i]);
                        const float act = p.activation == 0 ? g / (1.0f + expf(-g)) : p.activation == 1 ? 0.5f * g * (1.0f + erff(g * 0.70710678118654752440f)) : g;
                        result[i] = __float2bfloat16_rn(__bfloat162float(up[i]) * __bfloat162float(__float2bfloat16_rn(act)));
                    }
                    __nv_bfloat16* destination = static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(token) * p.hidden + row0 + part * 8;
                    if (p.hidden % 8 == 0 && row0 + kTcRows / 2 <= p.hidden) {
                        *reinterpret_cast<uint4*>(destination) = *reinterpret_cast<const uint4*>(result);
                    } else {
                        for (int i = 0; i < 8; ++i)
                            if (row0 + part * 8 + i < p.hidden) destination[i] = result[i];
                    }
                }
            } else if (as_bfloat16) {
                // 16 pieces of 8 rows per token
                for (int piece = epilogue_thread; piece < BN * 16; piece += 128) {
                    const int token_local = piece >> 4, part = piece & 15;
                    const int token = token0 + token_local;
                    if (token >= p.tokens) continue;
                    const __nv_bfloat16* source = reinterpret_cast<const __nv_bfloat16*>(tiles) + token_local * kPitchHalf + part * 8;
                    __nv_bfloat16* destination = static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(token) * p.n + row0 + part * 8;
                    if (vector_ok) {
                        *reinterpret_cast<uint4*>(destination) = *reinterpret_cast<const uint4*>(source);
                    } else {
                        for (int i = 0; i < 8; ++i)
                            if (row0 + part * 8 + i < p.n) destination[i] = source[i];
                    }
                }
            } else {
                // 32 pieces of 4 rows per token
                for (int piece = epilogue_thread; piece < BN * 32; piece += 128) {
                    const int token_local = piece >> 5, part = piece & 31;
                    const int token = token0 + token_local;
                    if (token >= p.tokens) continue;
                    const float* source = reinterpret_cast<const float*>(tiles) + token_local * kPitchFloat + part * 4;
                    const size_t token_row = p.epilogue == kTcPartial ? static_cast<size_t>(blockIdx.z) * p.tokens + token : static_cast<size_t>(token);
                    float* destination = static_cast<float*>(p.out) + token_row * p.n + row0 + part * 4;
                    float4 value = *reinterpret_cast<const float4*>(source);
                    if (p.epilogue == kTcResidualAdd) {
                        value.x = __bfloat162float(__float2bfloat16_rn(value.x));
                        value.y = __bfloat162float(__float2bfloat16_rn(value.y));
                        value.z = __bfloat162float(__float2bfloat16_rn(value.z));
                        value.w = __bfloat162float(__float2bfloat16_rn(value.w));
                    }
                    if (p.n % 4 == 0 && row0 + kTcRows <= p.n) {
                        if (p.epilogue == kTcResidualAdd) {
                            const float4 old = *reinterpret_cast<const float4*>(destination);
                            value.x += old.x;
                            value.y += old.y;
                            value.z += old.z;
                            value.w += old.w;
                        }
                        *reinterpret_cast<float4*>(destination) = value;
                    } else {
                        const float parts[4] = {value.x, value.y, value.z, value.w};
                        for (int i = 0; i < 4; ++i)
                            if (row0 + part * 4 + i < p.n) destination[i] = p.epilogue == kTcResidualAdd ? destination[i] + parts[i] : parts[i];
                    }
                }
            }
        }
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kColumns) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// The same product for many tokens (prefill): tiles of 128 rows of W x 256 tokens, one CTA per SM that
// walks tiles m + n * m_tiles in steps of the grid, and two accumulators in tensor memory, so that the
// epilogue of a tile (tensor memory -> registers -> the output, by eight warps) runs while the
// products of the next tile are issued.  All of K per tile; epilogues as above except the partial one.
// ---------------------------------------------------------------------------------------------
// Tiles of 256 tokens (four stages of 48 KB), 128 (six of 32 KB) or 64 (eight of 24 KB): 192 KB of
// stages each way.  PAIR: two CTAs of a cluster share a tile of 256 rows of W x 256 tokens; each loads
// its 128 rows of W and its 128 tokens of X (six stages of 32 KB), and the even CTA issues products over
// both CTAs' shared and tensor memory (cta_group::2).  A CTA then fetches 32 KB for every 128 x 256 x 64
// product instead of 48 KB: measured 4 to 6 % faster where a launch has several rounds of tiles, as much
// slower where it has one (the launcher chooses).
template <int BN, bool PAIR>
struct PersistShape {
    static_assert(BN == 64 || BN == 128 || BN == 256, "tiles of 64, 128 or 256 tokens");
    static_assert(!PAIR || BN == 256, "a pair of CTAs takes tiles of 256 tokens");
    static constexpr int kXTokens = PAIR ? BN / 2 : BN;   // tokens of X a CTA loads per stage
    static constexpr int kStageBytes = kTcRows * kTcBlockK * 2 + kXTokens * kTcBlockK * 2;
    static constexpr int kStages = 4 * 48 * 1024 / kStageBytes;
    static_assert(kStages * kStageBytes == 4 * 48 * 1024 && kStages <= 8, "the stages fill 192 KB");
};
constexpr int kPersistExchangePitch = 80;   // bytes a thread's 32 activated gates take (64) and 16 to spread the banks
constexpr int kPersistRegionBytes = 16 * 1024;   // per half of the epilogue: two output buffers of 8 KB, or (gated) two of 4 KB and the exchange
constexpr int kPersistExchangeBytes = 2 * kPersistRegionBytes;
static_assert(4 * 2 * 32 * kPersistExchangePitch <= kPersistExchangeBytes, "the padded exchange of the path without bulk stores fits too");
constexpr int kPersistThreads = 64 + 256;   // producer warp, issuer warp, eight epilogue warps
constexpr int kPersistSharedBytes = 4 * 48 * 1024 + kPersistExchangeBytes + 1024 + 256;
static_assert((2 * 8 + 4) * 8 + 4 <= 256, "the barriers of the deepest ring fit behind the exchange");

template <int BN, bool PAIR>
__global__ void __launch_bounds__(kPersistThreads)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                               const __grid_constant__ CUtensorMap map_out, const TcParams p, int m_tiles, int n_tiles, int slices) {
    constexpr int STAGES = PersistShape<BN, PAIR>::kStages, kPersistStageBytes = PersistShape<BN, PAIR>::kStageBytes;
    constexpr int kXTokens = PersistShape<BN, PAIR>::kXTokens;
    // With PAIR the walkers are the pairs: `walker` of `walkers`, and `rank` within the pair; m_tiles
    // counts tiles of both CTAs' rows.
    const int rank = PAIR ? static_cast<int>(cluster_rank()) : 0;
    const int walker = PAIR ? static_cast<int>(blockIdx.x) >> 1 : static_cast<int>(blockIdx.x);
    const int walkers = PAIR ? static_cast<int>(gridDim.x) >> 1 : static_cast<int>(gridDim.x);
    allow_next_kernel();   // its CTAs find room as this kernel's CTAs finish: the tails overlap
    constexpr int kWBytes = kTcRows * kTcBlockK * 2;
    extern __shared__ unsigned char raw_shared[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_shared) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* exchange = tiles + STAGES * kPersistStageBytes;
    uint64_t* barriers = reinterpret_cast<uint64_t*>(exchange + kPersistExchangeBytes);
    uint64_t* full = barriers;                      // [STAGES]
    uint64_t* empty = barriers + STAGES;            // [STAGES]
    uint64_t* tmem_full = barriers + 2 * STAGES;    // [2] an accumulator is complete
    uint64_t* tmem_empty = barriers + 2 * STAGES + 2;   // [2] an accumulator has been read out
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(barriers + 2 * STAGES + 4);
    __shared__ int failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool gated = p.epilogue == kTcGated;
    const int rows_per_cta = gated ? kTcRows / 2 : kTcRows;
    const int rows_per_tile = PAIR ? 2 * rows_per_cta : rows_per_cta;
    const int k_blocks = (p.k + kTcBlockK - 1) / kTcBlockK;
    const int num_tiles = m_tiles * n_tiles;
    // With K slices a walker's items are (tile, slice) pairs, item = slice * num_tiles + tile: a slice's
    // blocks of K are first_block(slice) ... + block_count(slice) - 1, and its sums go to the slice's own
    // [tokens, n] of float32 (kTcPartial).
    const int num_items = num_tiles * slices;
    auto first_block = [&](int item) { return (item / num_tiles) * p.blocks_per_slice; };
    auto block_count = [&](int item) { return min(p.blocks_per_slice, k_blocks - first_block(item)); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            barrier_init(&full[s], 1);    // PAIR: only the even CTA's are used, for both CTAs' bytes
            barrier_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            barrier_init(&tmem_full[a], 1);
            barrier_init(&tmem_empty[a], PAIR ? 16 : 8);   // one arrival per epilogue warp (PAIR: of both CTAs, at the even one)
        }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_address(tmem_slot)), "r"(2 * BN) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_address(tmem_slot)), "r"(2 * BN) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if constexpr (PAIR) cluster_sync();   // the partner's barriers exist before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // The weights do not depend on the kernel before this one (which may still be running: this
        // kernel is launched to start early): the first stages ask for their tiles of W at once, and
        // only the tiles of X wait for that kernel.  PAIR: both CTAs load, each its rows and its
        // tokens; all bytes count on the even CTA's barrier, which that CTA arms.
        int issued = 0;
        bool ok = true;
        const int early = walker < num_items ? min(STAGES, block_count(walker)) : 0;
        auto arm = [&](int s) {
            if (rank == 0) barrier_expect(&full[s], (PAIR ? 2 : 1) * kPersistStageBytes);
        };
        auto load = [&](unsigned char* destination, const CUtensorMap* map, int x, int y, int s) {
            if constexpr (PAIR) tma_load_2d_pair(destination, map, x, y, cluster_address(&full[s], 0));
            else tma_load_2d(destination, map, x, y, &full[s]);
        };
        for (int block = 0; block < early; ++block) {
            const int row0 = ((walker % num_tiles) % m_tiles) * rows_per_tile + rank * rows_per_cta;
            const int column = (first_block(walker) + block) * kTcBlockK;
            arm(block);
            load(tiles + block * kPersistStageBytes, &map_w, column, row0, block);
            if (gated) load(tiles + block * kPersistStageBytes + kWBytes / 2, &map_w, column, p.hidden + row0, block);
        }
        wait_for_previous_kernel();
        for (int block = 0; block < early; ++block)
            load(tiles + block * kPersistStageBytes + kWBytes, &map_x, (first_block(walker) + block) * kTcBlockK, ((walker % num_tiles) / m_tiles) * BN + rank * kXTokens, block);
        issued = early;
        for (int item = walker; item < num_items && ok; item += walkers) {
            const int tile = item % num_tiles;
            const int row0 = (tile % m_tiles) * rows_per_tile + rank * rows_per_cta, token0 = (tile / m_tiles) * BN + rank * kXTokens;
            const int first = first_block(item), count = block_count(item);
            for (int block = item == walker ? early : 0; block < count; ++block, ++issued) {
                const int s = issued % STAGES, round = issued / STAGES;
                if (round > 0 && !barrier_wait(&empty[s], (round - 1) & 1)) {
                    atomicExch(&failed, 1);
                    ok = false;
                    break;
                }
                unsigned char* stage = tiles + s * kPersistStageBytes;
                arm(s);
                const int column = (first + block) * kTcBlockK;
                load(stage, &map_w, column, row0, s);
                if (gated) load(stage + kWBytes / 2, &map_w, column, p.hidden + row0, s);
                load(stage + kWBytes, &map_x, column, token0, s);
            }
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        constexpr uint32_t idesc = PAIR ? instruction_descriptor_pair<BN>() : instruction_descriptor<BN>();
        int consumed = 0, local = 0;
        bool ok = true;
        for (int item = walker; item < num_items && ok; item += walkers, ++local) {
            const int accumulator = local & 1, use = local >> 1;
            if (use > 0 && !barrier_wait(&tmem_empty[accumulator], (use - 1) & 1)) {
                atomicExch(&failed, 1);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(accumulator * BN);
            const int count = block_count(item);
            for (int block = 0; block < count; ++block, ++consumed) {
                const int s = consumed % STAGES, round = consumed / STAGES;
                if (!barrier_wait(&full[s], round & 1)) {
                    atomicExch(&failed, 1);
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                unsigned char* stage = tiles + s * kPersistStageBytes;
                const uint64_t desc_w = tile_descriptor(stage), desc_x = tile_descriptor(stage + kWBytes);
#pragma unroll
                for (int k = 0; k < kTcBlockK / 16; ++k) {
                    if constexpr (PAIR) mma_f16_pair(tmem_d, desc_w + 2 * k, desc_x + 2 * k, idesc, block > 0 || k > 0);
                    else mma_f16(tmem_d, desc_w + 2 * k, desc_x + 2 * k, idesc, block > 0 || k > 0);
                }
                if constexpr (PAIR) mma_commit_pair(&empty[s]);
                else mma_commit(&empty[s]);
            }
            if (ok) {
                if constexpr (PAIR) mma_commit_pair(&tmem_full[accumulator]);
                else mma_commit(&tmem_full[accumulator]);
            }
        }
    } else if (warp >= 2) {
        // Eight warps: warp & 3 is the quarter of the accumulator's lanes a warp may read, and each
        // half of the 256 tokens has four warps.  A thread holds one row of W for 32 tokens at a time
        // and writes them itself: for one token a warp's 32 rows are one piece of 128 (float32) or
        // 64 (bfloat16) bytes in the output, so that nothing has to be turned in shared memory.
        wait_for_previous_kernel();   // before anything of the output is read or written
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int half_barrier = 5 + half;   // 1..4 belong to the pairs of warps of the gated epilogue
        const bool issuer = quarter == 0 && lane == 0;
        unsigned char* region = exchange + half * kPersistRegionBytes;
        int local = 0, groups = 0;
        for (int item = walker; item < num_items; item += walkers, ++local) {
            const int accumulator = local & 1, use = local >> 1;
            const int tile = item % num_tiles, slice = item / num_tiles;
            const int row0 = (tile % m_tiles) * rows_per_tile + rank * rows_per_cta, token0 = (tile / m_tiles) * BN + half * (BN / 2);
            uint32_t arrived = barrier_wait(&tmem_full[accumulator], use & 1) ? 1u : 0u;
            {
                // Warps that meet at named barriers below go on together or not at all.
                uint32_t all;
                asm volatile(
                    "{\n"
                    ".reg .pred mine, all;\n"
                    "setp.ne.u32 mine, %1, 0;\n"
                    "bar.red.and.pred all, %2, 128, mine;\n"
                    "selp.u32 %0, 1, 0, all;\n"
                    "}\n"
                    : "=r"(all)
                    : "r"(arrived), "r"(half_barrier)
                    : "memory");
                arrived = all;
            }
            if (!arrived) {
                atomicExch(&failed, 1);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(accumulator * BN + half * (BN / 2)) + (static_cast<uint32_t>(quarter * 32) << 16);
            // Where the output's rows are 16-byte aligned it leaves by bulk tensor stores: the four
            // warps of a half set 32 tokens (16 of float32) x 128 rows down in shared memory, token by
            // token as the output has them, and one thread sends the box off.  Stores issued by the
            // threads themselves queue behind the loads of the stages and took longer than a tile's
            // products.  Onto the residual stream the box is added in the memory system.
            const bool wide = p.epilogue == kTcStoreFloat || p.epilogue == kTcResidualAdd || p.epilogue == kTcPartial;
            const int step = wide ? 16 : 32;
#pragma unroll 1
            for (int column = 0; p.bulk_store && column < BN / 2; column += step, ++groups) {
                if (token0 + column >= p.tokens) break;   // the same for the whole half
                unsigned char* out_buffer = region + (groups & 1) * (gated ? 4096 : 8192);
                // the store before last, which read this buffer, has read it
                if (issuer) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                named_barrier(half_barrier, 128);
                if (wide) {
                    uint32_t v[16];
                    tmem_load_16(tmem_d + static_cast<uint32_t>(column), v);
                    float* stage = reinterpret_cast<float*>(out_buffer) + quarter * 32 + lane;
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        stage[i * kTcRows] = p.epilogue == kTcResidualAdd ? __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[i]))) : __uint_as_float(v[i]);
                } else if (!gated) {
                    uint32_t v[32];
                    tmem_load_32(tmem_d + static_cast<uint32_t>(column), v);
                    __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(out_buffer) + quarter * 32 + lane;
#pragma unroll
                    for (int i = 0; i < 32; ++i) stage[i * kTcRows] = __float2bfloat16_rn(__uint_as_float(v[i]));
                } else {
                    // Lanes 0-63 of the accumulator are rows of `up`, lanes 64-127 the same rows of `gate`:
                    // the warp with the gates activates them and hands them over (two buffers, a barrier
                    // of the two warps); the warp with `up` multiplies.  16-byte pieces, swizzled by lane.
                    uint32_t v[32];
                    tmem_load_32(tmem_d + static_cast<uint32_t>(column), v);
                    unsigned char* handover = region + 8192 + ((quarter & 1) * 2 + (groups & 1)) * 2048 + lane * 64;
                    const int pair_barrier = 1 + half * 2 + (quarter & 1);
                    if (quarter >= 2) {
#pragma unroll
                        for (int piece = 0; piece < 4; ++piece) {
                            uint4 packed;
                            __nv_bfloat162* halves = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                float act[2];
#pragma unroll
                                for (int e = 0; e < 2; ++e) {
                                    const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[piece * 8 + 2 * i + e])));
                                    act[e] = p.activation == 0 ? __fdividef(g, 1.0f + __expf(-g)) : p.activation == 1 ? 0.5f * g * (1.0f + erff(g * 0.70710678118654752440f)) : g;
                                }
                                halves[i] = __floats2bfloat162_rn(act[0], act[1]);
                            }
                            *reinterpret_cast<uint4*>(handover + ((piece ^ (lane >> 1)) & 3) * 16) = packed;
                        }
                        named_barrier(pair_barrier, 64);
                    } else {
                        named_barrier(pair_barrier, 64);
                        __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(out_buffer) + quarter * 32 + lane;
#pragma unroll
                        for (int piece = 0; piece < 4; ++piece) {
                            const uint4 packed = *reinterpret_cast<const uint4*>(handover + ((piece ^ (lane >> 1)) & 3) * 16);
                            const __nv_bfloat162* halves = reinterpret_cast<const __nv_bfloat162*>(&packed);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float2 act = __bfloat1622float2(halves[i]);
                                const int token = piece * 8 + 2 * i;
                                const float up0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[token])));
                                const float up1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[token + 1])));
                                stage[token * (kTcRows / 2)] = __float2bfloat16_rn(up0 * act.x);
                                stage[(token + 1) * (kTcRows / 2)] = __float2bfloat16_rn(up1 * act.y);
                            }
                        }
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // what the threads wrote, seen by the bulk store
                named_barrier(half_barrier, 128);
                if (issuer) {
                    if (p.epilogue == kTcPartial) bulk_store_3d(&map_out, out_buffer, row0, token0 + column, slice);
                    else bulk_store_2d(&map_out, out_buffer, row0, token0 + column, p.epilogue == kTcResidualAdd);
                }
            }
#pragma unroll 1
            for (int column = 0; !p.bulk_store && column < BN / 2; column += 32) {
                if (token0 + column >= p.tokens) break;   // the same for the whole warp
                uint32_t v[32];
                tmem_load_32(tmem_d + static_cast<uint32_t>(column), v);
                const int tokens_here = min(32, p.tokens - token0 - column);
                if (gated) {
                    // Lanes 0-63 of the accumulator are rows of `up`, lanes 64-127 the same rows of
                    // `gate`.  The warp with the gates activates them and hands them over in shared
                    // memory (two buffers, one named barrier of 64 threads per group of 32 tokens);
                    // the warp with `up` multiplies and writes.
                    unsigned char* buffer = exchange + ((half * 2 + (quarter & 1)) * 2 + ((column >> 5) & 1)) * 32 * kPersistExchangePitch;
                    uint4* mine = reinterpret_cast<uint4*>(buffer + lane * kPersistExchangePitch);
                    const int pair_barrier = 1 + half * 2 + (quarter & 1);
                    if (quarter >= 2) {
#pragma unroll
                        for (int piece = 0; piece < 4; ++piece) {
                            uint4 packed;
                            __nv_bfloat162* halves = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                float act[2];
#pragma unroll
                                for (int e = 0; e < 2; ++e) {
                                    const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[piece * 8 + 2 * i + e])));
                                    // exp and the division by fast hardware approximations (a few units in the
                                    // last place of float32, far below the bfloat16 rounding that follows)
                                    act[e] = p.activation == 0 ? __fdividef(g, 1.0f + __expf(-g)) : p.activation == 1 ? 0.5f * g * (1.0f + erff(g * 0.70710678118654752440f)) : g;
                                }
                                halves[i] = __floats2bfloat162_rn(act[0], act[1]);
                            }
                            mine[piece] = packed;
                        }
                        asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier) : "memory");
                    } else {
                        asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier) : "memory");
                        const int row = row0 + quarter * 32 + lane;
                        __nv_bfloat16* destination = static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(token0 + column) * p.hidden + row;
                        const bool whole = tokens_here == 32;
                        if (row < p.hidden) {
#pragma unroll
                            for (int piece = 0; piece < 4; ++piece) {
                                const uint4 packed = mine[piece];
                                const __nv_bfloat162* halves = reinterpret_cast<const __nv_bfloat162*>(&packed);
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const float2 act = __bfloat1622float2(halves[i]);
                                    const int token = piece * 8 + 2 * i;
                                    const float up0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[token])));
                                    const float up1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[token + 1])));
                                    if (whole || token < tokens_here) destination[static_cast<size_t>(token) * p.hidden] = __float2bfloat16_rn(up0 * act.x);
                                    if (whole || token + 1 < tokens_here) destination[static_cast<size_t>(token + 1) * p.hidden] = __float2bfloat16_rn(up1 * act.y);
                                }
                            }
                        }
                    }
                } else {
                    const int row = row0 + quarter * 32 + lane;
                    const bool whole = tokens_here == 32;
                    if (row < p.n) {
                        if (p.epilogue == kTcStore) {
                            __nv_bfloat16* destination = static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(token0 + column) * p.n + row;
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (whole || i < tokens_here) destination[static_cast<size_t>(i) * p.n] = __float2bfloat16_rn(__uint_as_float(v[i]));
                        } else if (p.epilogue == kTcStoreFloat || p.epilogue == kTcPartial) {
                            float* destination = static_cast<float*>(p.out) + (static_cast<size_t>(slice) * p.tokens + token0 + column) * p.n + row;
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (whole || i < tokens_here) destination[static_cast<size_t>(i) * p.n] = __uint_as_float(v[i]);
                        } else {
                            // All 32 loads of the residual stream leave before the first sum is stored.
                            float* destination = static_cast<float*>(p.out) + static_cast<size_t>(token0 + column) * p.n + row;
                            float old[32];
#pragma unroll
                            for (int i = 0; i < 32; ++i) old[i] = whole || i < tokens_here ? destination[static_cast<size_t>(i) * p.n] : 0.0f;
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (whole || i < tokens_here)
                                    destination[static_cast<size_t>(i) * p.n] = old[i] + __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[i])));
                        }
                    }
                }
            }
            // The accumulator has been read out: the issuer may reuse it for the tile after next.
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                if constexpr (PAIR) barrier_arrive_cluster(cluster_address(&tmem_empty[accumulator], 0));
                else barrier_arrive(&tmem_empty[accumulator]);
            }
        }
        if (issuer) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (failed) {
        if (threadIdx.x == 0) report_error(p.status, kWaitTimeout);
        for (int spin = 0; spin < 2000; ++spin) __nanosleep(1000);
        __syncthreads();
    }
    // PAIR: neither CTA leaves, or gives its tensor memory back, while the other may still touch them.
    if constexpr (PAIR) cluster_sync();
    if (warp == 1) {
        if constexpr (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
    }
}

// One thread waits, for at most `nanoseconds`, on a barrier that nothing arrives on, and reports the
// wait that gave up the way the products do: what the host sees of a lost arrival, without losing one.
__global__ void wait_probe_kernel(int* status, unsigned long long nanoseconds) {
    __shared__ uint64_t barrier;
    barrier_init(&barrier, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!barrier_wait(&barrier, 0, nanoseconds)) report_error(status, kWaitTimeout);
}

// out = epilogue(sum over slices of partials[slice]), slices added in order.  VEC elements per thread.
template <int VEC>
__global__ void gemm_tcgen05_reduce_kernel(const float* __restrict__ partials, void* __restrict__ out, size_t count, int slices, int epilogue) {
    const size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC;
    wait_for_previous_kernel();   // launched to start early: the partial sums are its predecessor's
    allow_next_kernel();
    if (i >= count) return;
    float sum[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) sum[e] = 0.0f;
    for (int s = 0; s < slices; ++s) {
        const float* source = partials + static_cast<size_t>(s) * count + i;
        if constexpr (VEC == 4) {
            const float4 v = *reinterpret_cast<const float4*>(source);
            sum[0] += v.x, sum[1] += v.y, sum[2] += v.z, sum[3] += v.w;
        } else {
            sum[0] += source[0];
        }
    }
    if (epilogue == kTcStore) {
        __nv_bfloat16* destination = static_cast<__nv_bfloat16*>(out) + i;
        if constexpr (VEC == 4) {
            const __nv_bfloat162 low = __floats2bfloat162_rn(sum[0], sum[1]), high = __floats2bfloat162_rn(sum[2], sum[3]);
            uint2 packed;
            packed.x = *reinterpret_cast<const uint32_t*>(&low);
            packed.y = *reinterpret_cast<const uint32_t*>(&high);
            *reinterpret_cast<uint2*>(destination) = packed;
        } else {
            destination[0] = __float2bfloat16_rn(sum[0]);
        }
    } else if (epilogue == kTcStoreFloat) {
        float* destination = static_cast<float*>(out) + i;
        if constexpr (VEC == 4) *reinterpret_cast<float4*>(destination) = make_float4(sum[0], sum[1], sum[2], sum[3]);
        else destination[0] = sum[0];
    } else {
        float* destination = static_cast<float*>(out) + i;
        if constexpr (VEC == 4) {
            float4 v = *reinterpret_cast<const float4*>(destination);
            v.x += __bfloat162float(__float2bfloat16_rn(sum[0]));
            v.y += __bfloat162float(__float2bfloat16_rn(sum[1]));
            v.z += __bfloat162float(__float2bfloat16_rn(sum[2]));
            v.w += __bfloat162float(__float2bfloat16_rn(sum[3]));
            *reinterpret_cast<float4*>(destination) = v;
        } else {
            destination[0] += __bfloat162float(__float2bfloat16_rn(sum[0]));
        }
    }
}

// A [rows, k] bfloat16 row-major matrix seen through boxes of [box_rows, 64] with 128-byte swizzle;
// what lies outside the matrix reads as zero.
static bool make_map(CUtensorMap* map, const void* base, int rows, int k, int box_rows) {
    EncodeTiled encode = encode_tiled();
    if (encode == nullptr) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
    const cuuint32_t box[2] = {kTcBlockK, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t element_strides[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int STAGES>
int launch_tcgen05_variant(const CUtensorMap& map_w, const CUtensorMap& map_x, const TcParams& p, dim3 grid, cudaStream_t stream) {
    using Shared = TcShared<BN, STAGES>;
    auto kernel = gemm_tcgen05_kernel<BN, STAGES>;
    static OncePerDevice configured;
    if (allow_shared_memory(configured, kernel, Shared::kBytes) != cudaSuccess) return static_cast<int>(cudaGetLastError());
    // Launched so that it may start while the kernel before it still runs (it waits for that kernel
    // itself, after its first tiles of W are on their way).
    return static_cast<int>(launch_overlapped(kernel, grid, dim3(kTcThreads), Shared::kBytes, stream, map_w, map_x, p));
}

template <int BN>
int launch_tcgen05(const CUtensorMap& map_w, const void* x, TcParams p, int slices, cudaStream_t stream) {
    const int rows_per_cta = p.epilogue == kTcGated ? kTcRows / 2 : kTcRows;
    const int row_extent = p.epilogue == kTcGated ? p.hidden : p.n;
    CUtensorMap map_x;
    if (!make_map(&map_x, x, p.tokens, p.k, BN)) return -5;
    const dim3 grid((row_extent + rows_per_cta - 1) / rows_per_cta, (p.tokens + BN - 1) / BN, slices);
    // About 100 KB of stages lets two CTAs share an SM, so that one's epilogue hides behind the other's
    // products.  A grid that does not even fill the SMs once gets all of an SM's shared memory instead:
    // what bounds it is how many bytes of W it keeps in flight.
    constexpr int shallow = BN <= 32 ? 5 : (BN <= 64 ? 4 : 3);
    constexpr int deep = BN <= 32 ? 10 : (BN <= 64 ? 8 : 6);
    if (static_cast<int>(grid.x * grid.y * grid.z) <= multiprocessor_count()) return launch_tcgen05_variant<BN, deep>(map_w, map_x, p, grid, stream);
    return launch_tcgen05_variant<BN, shallow>(map_w, map_x, p, grid, stream);
}

// The output [tokens, width] seen through boxes of [box_tokens, box_width], laid down in shared memory row after row.
static bool make_out_map(CUtensorMap* map, void* base, int tokens, int width, bool is_float, int box_width, int box_tokens) {
    EncodeTiled encode = encode_tiled();
    if (encode == nullptr) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(width), static_cast<cuuint64_t>(tokens)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(width) * (is_float ? 4 : 2)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_width), static_cast<cuuint32_t>(box_tokens)};
    const cuuint32_t element_strides[2] = {1, 1};
    return encode(map, is_float ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, element_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The K slices' partial sums [slices, tokens, width] of float32 seen through boxes of [1, box_tokens, box_width]:
// a box that reaches past a slice's last token is cut there.
static bool make_partial_map(CUtensorMap* map, void* base, int slices, int tokens, int width, int box_width, int box_tokens) {
    EncodeTiled encode = encode_tiled();
    if (encode == nullptr) return false;
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(width), static_cast<cuuint64_t>(tokens), static_cast<cuuint64_t>(slices)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(width) * 4, static_cast<cuuint64_t>(width) * 4 * static_cast<cuuint64_t>(tokens)};
    const cuuint32_t box[3] = {static_cast<cuuint32_t>(box_width), static_cast<cuuint32_t>(box_tokens), 1};
    const cuuint32_t element_strides[3] = {1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, bool PAIR>
int launch_persistent(const CUtensorMap& map_w, const void* x, TcParams p, int m_tiles, int sms, int slices, cudaStream_t stream) {
    CUtensorMap map_x;
    if (!make_map(&map_x, x, p.tokens, p.k, PersistShape<BN, PAIR>::kXTokens)) return -5;
    const bool is_partial = p.epilogue == kTcPartial;
    const bool is_float = p.epilogue == kTcStoreFloat || p.epilogue == kTcResidualAdd || is_partial, is_gated = p.epilogue == kTcGated;
    const int width = is_gated ? p.hidden : p.n;
    CUtensorMap map_out = map_x;   // not read unless the output leaves by bulk stores
    p.bulk_store = (static_cast<size_t>(width) * (is_float ? 4 : 2)) % 16 == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 ? 1 : 0;
    if (p.bulk_store && is_partial && !make_partial_map(&map_out, p.out, slices, p.tokens, width, kTcRows, 16)) return -5;
    if (p.bulk_store && !is_partial && !make_out_map(&map_out, p.out, p.tokens, width, is_float, is_gated ? kTcRows / 2 : kTcRows, is_float ? 16 : 32)) return -5;
    auto kernel = gemm_tcgen05_persistent_kernel<BN, PAIR>;
    static OncePerDevice configured;
    if (allow_shared_memory(configured, kernel, kPersistSharedBytes) != cudaSuccess) return static_cast<int>(cudaGetLastError());
    const int n_tiles = (p.tokens + BN - 1) / BN;
    const int items = m_tiles * n_tiles * slices;
    if constexpr (!PAIR) {
        const int grid = items < sms ? items : sms;
        return static_cast<int>(launch_overlapped(kernel, dim3(grid), dim3(kPersistThreads), kPersistSharedBytes, stream, map_w, map_x, map_out, p, m_tiles, n_tiles, slices));
    } else {
        // m_tiles counts the pairs' tiles of 256 (gated: 128) rows; a cluster of two CTAs per walker.
        const int pairs = items < sms / 2 ? items : sms / 2;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(2 * pairs);
        config.blockDim = dim3(kPersistThreads);
        config.dynamicSmemBytes = kPersistSharedBytes;
        config.stream = stream;
        cudaLaunchAttribute attributes[2];
        attributes[0].id = cudaLaunchAttributeClusterDimension;
        attributes[0].val.clusterDim.x = 2;
        attributes[0].val.clusterDim.y = 1;
        attributes[0].val.clusterDim.z = 1;
        attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attributes[1].val.programmaticStreamSerializationAllowed = overlap_launches() ? 1 : 0;
        config.attrs = attributes;
        config.numAttrs = 2;
        return static_cast<int>(cudaLaunchKernelEx(&config, kernel, map_w, map_x, map_out, p, m_tiles, n_tiles, slices));
    }
}

}  // namespace lb

extern "C" {

int lb_sum_slices(const float* scratch, void* out, int tokens, int n, int slices, int epilogue, cudaStream_t stream);

// Runs the bounded wait of the tcgen05 kernels on a barrier that is never completed: it gives up after
// `nanoseconds` (at most a tenth of a second here) and writes the timeout code to `status`.
int lb_tcgen05_wait_probe(int* status, long long nanoseconds, cudaStream_t stream) {
    if (nanoseconds < 0 || nanoseconds > 100000000ll) return -2;
    lb::wait_probe_kernel<<<1, 1, 0, stream>>>(status, static_cast<unsigned long long>(nanoseconds));
    return static_cast<int>(cudaGetLastError());
}

// Floats of scratch a call with `slices` K slices needs (0 for one slice).
long long lb_gemm_tcgen05_scratch_floats(int tokens, int n, int slices) {
    return slices > 1 ? static_cast<long long>(slices) * tokens * n : 0;
}

// epilogue: 0 bfloat16 store, 1 float32 store, 2 add to the float32 residual stream, 4 gated: w is
// [n, k] with n = 2 * hidden, rows [up ; gate], out is [tokens, hidden] = up * act(gate) (one K slice).
// Returns 0, a CUDA error, -2 for sizes the kernel does not take (k % 8 != 0: rows must be 16-byte
// aligned; tokens < 1), -3 if the scratch is too small, -5 if no tensor map could be made.
// defer_sum: with more than one slice, leave the partial sums in `scratch` ([slices][tokens][n]) for the
// caller (lb_sum_slices, or a consumer that adds them itself); `out` is not touched then.
int lb_gemm_tcgen05(const void* x, const void* w, void* out, float* scratch, long long scratch_floats, int tokens, int k, int n, int epilogue,
                    int activation, int slices, int defer_sum, int* status, cudaStream_t stream) {
    if (tokens < 1 || n < 1 || k < 8 || k % 8 != 0 || epilogue < 0 || epilogue == 3 || epilogue > 4) return -2;
    if (epilogue == lb::kTcGated) {
        if (n % 2 != 0) return -2;
        slices = 1;
    }
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return -2;
    const int total_blocks = (k + lb::kTcBlockK - 1) / lb::kTcBlockK;
    slices = max(1, min(slices, total_blocks));
    lb::TcParams p;
    p.tokens = tokens;
    p.n = n;
    p.k = k;
    p.blocks_per_slice = (total_blocks + slices - 1) / slices;
    slices = (total_blocks + p.blocks_per_slice - 1) / p.blocks_per_slice;
    p.status = status;
    p.hidden = n / 2;
    p.activation = activation;
    p.bulk_store = 0;
    p.early_successor = tokens > 16 ? 1 : 0;
    if (slices > 1) {
        if (scratch == nullptr || lb_gemm_tcgen05_scratch_floats(tokens, n, slices) > scratch_floats) return -3;
        p.out = scratch;
        p.epilogue = lb::kTcPartial;
    } else {
        p.out = out;
        p.epilogue = epilogue;
    }
    CUtensorMap map_w;
    if (!lb::make_map(&map_w, w, n, k, epilogue == lb::kTcGated ? lb::kTcRows / 2 : lb::kTcRows)) return -5;
    int code;
    if (tokens > 128 && slices == 1) {
        // Many tokens: one CTA (or pair of CTAs) per SM walks the tiles.
        const int sms = lb::multiprocessor_count();
        const int rows_per_tile = epilogue == lb::kTcGated ? lb::kTcRows / 2 : lb::kTcRows;
        const int row_extent = epilogue == lb::kTcGated ? p.hidden : n;
        const int m_tiles = (row_extent + rows_per_tile - 1) / rows_per_tile;
        // Which tile: measured, a round of tiles takes about as long whatever the tile's width while one
        // round is all there is (what bounds it is a CTA's walk through K), so the narrowest tile that
        // still needs one round only wins there; beyond one round a 128-token tile takes 0.72 of the
        // time of a 256-token one and pays only where it saves whole rounds.  A pair of CTAs on tiles
        // of 256 rows x 256 tokens is 4 to 6 % faster where there is much work per launch, and slower
        // by as much where there is little.
        const int tiles_64 = m_tiles * ((tokens + 63) / 64), tiles_128 = m_tiles * ((tokens + 127) / 128), tiles_256 = m_tiles * ((tokens + 255) / 256);
        const int wide_cost = 2 * ((tiles_256 + sms - 1) / sms), narrow_cost = (tiles_128 + sms - 1) / sms;
        const long long work = static_cast<long long>(tiles_256) * ((k + lb::kTcBlockK - 1) / lb::kTcBlockK);
        int tile = tiles_64 <= sms ? 64 : tiles_128 <= sms ? 128 : narrow_cost * 18 < wide_cost * 25 / 2 ? 128 : 256;
        if (tile == 256 && (epilogue == lb::kTcGated || work >= 12000)) tile = 512;   // the pair
        if (const char* forced = getenv("LALAMO_B200_TCGEN05_TILE")) tile = atoi(forced);
        if (tile == 512) return lb::launch_persistent<256, true>(map_w, x, p, (m_tiles + 1) / 2, sms, 1, stream);
        if (tile == 64) return lb::launch_persistent<64, false>(map_w, x, p, m_tiles, sms, 1, stream);
        if (tile == 128) return lb::launch_persistent<128, false>(map_w, x, p, m_tiles, sms, 1, stream);
        return lb::launch_persistent<256, false>(map_w, x, p, m_tiles, sms, 1, stream);
    }
    static const bool walk_slices = []() {
        const char* setting = getenv("LALAMO_B200_TCGEN05_WALK_SLICES");
        return setting == nullptr || setting[0] != '0';
    }();
    if (tokens > 128 && walk_slices) {
        // Many tokens and few tiles: tiles of 256 tokens (a tile of 128 x 128 asks L2 for a byte per 64
        // operations, which bounds it at half of what the tensor cores do), with K cut so that the tiles
        // times the slices fill the SMs.
        const int sms = lb::multiprocessor_count();
        const int m_tiles = (n + lb::kTcRows - 1) / lb::kTcRows;
        int tile = 256;
        if (const char* forced = getenv("LALAMO_B200_TCGEN05_TILE")) tile = atoi(forced);
        if (tile == 512) code = lb::launch_persistent<256, true>(map_w, x, p, (m_tiles + 1) / 2, sms, slices, stream);
        else if (tile == 128) code = lb::launch_persistent<128, false>(map_w, x, p, m_tiles, sms, slices, stream);
        else code = lb::launch_persistent<256, false>(map_w, x, p, m_tiles, sms, slices, stream);
        if (code != 0 || defer_sum) return code;
        return lb_sum_slices(scratch, out, tokens, n, slices, epilogue, stream);
    }
    if (tokens <= 32) code = lb::launch_tcgen05<32>(map_w, x, p, slices, stream);
    else if (tokens <= 64) code = lb::launch_tcgen05<64>(map_w, x, p, slices, stream);
    else code = lb::launch_tcgen05<128>(map_w, x, p, slices, stream);
    if (code != 0 || slices == 1 || defer_sum) return code;
    return lb_sum_slices(scratch, out, tokens, n, slices, epilogue, stream);
}

// out = epilogue(partials[0] + partials[1] + ...), the slices added in order; partials is [slices][tokens][n].
// epilogue: 0 bfloat16 store, 1 float32 store, 2 add (rounded to bfloat16 first) onto the float32 `out`.
int lb_sum_slices(const float* scratch, void* out, int tokens, int n, int slices, int epilogue, cudaStream_t stream) {
    if (tokens < 1 || n < 1 || slices < 1 || epilogue < 0 || epilogue > 2) return -2;
    const size_t count = static_cast<size_t>(tokens) * n;
    // Four elements a thread where the pointers allow 16-byte accesses (count % 4 == 0 keeps every slice aligned).
    if (count % 4 == 0 && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0)
        return static_cast<int>(lb::launch_overlapped(lb::gemm_tcgen05_reduce_kernel<4>, dim3(static_cast<unsigned>((count / 4 + 255) / 256)), dim3(256), 0, stream,
                                                      static_cast<const float*>(scratch), out, count, slices, epilogue));
    return static_cast<int>(lb::launch_overlapped(lb::gemm_tcgen05_reduce_kernel<1>, dim3(static_cast<unsigned>((count + 255) / 256)), dim3(256), 0, stream,
                                                  static_cast<const float*>(scratch), out, count, slices, epilogue));
}

}  // extern "C"
