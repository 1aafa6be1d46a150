// Token sampling on the device: logit processors in the reference's order
// (ban -> repetition -> presence -> frequency -> temperature -> top-k -> top-p -> min-p,
// lalamo/sampling.py:187-196), then a categorical draw by the Gumbel-max rule with a
// counter-based generator keyed per request, so a request's tokens do not depend on the batch.
//
// One block per row.  Top-k and top-p do not sort: they find the threshold value by a radix
// search over the order-preserving bit pattern of the 32-bit logits (four passes of eight bits)
// and settle ties by token index, as a stable descending sort would.
#include "common.cuh"

namespace lb {

constexpr int kSampleThreads = 1024;
constexpr int kMaxBanned = 16;

struct RowParams {
    float temperature;       // < 0: leave the logits as they are; 0: greedy
    int top_k;               // <= 0: off
    float top_p;             // >= 1: off
    float min_p;             // <= 0: off
    float repetition_penalty;   // 1: off
    float presence_penalty;     // 0: off
    float frequency_penalty;    // 0: off
    int count_slot;          // row of the token-count table, < 0: none
    unsigned seed_lo, seed_hi;
    unsigned draw;           // how many tokens this request has drawn before
    int banned[kMaxBanned];  // -1 terminated / padded
};

__device__ __forceinline__ unsigned order_key(float v) {
    const unsigned bits = __float_as_uint(v);
    return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

__device__ __forceinline__ void philox_round(unsigned (&ctr)[4], unsigned (&key)[2]) {
    const unsigned long long p0 = 0xD2511F53ull * ctr[0], p1 = 0xCD9E8D57ull * ctr[2];
    const unsigned hi0 = static_cast<unsigned>(p0 >> 32), lo0 = static_cast<unsigned>(p0);
    const unsigned hi1 = static_cast<unsigned>(p1 >> 32), lo1 = static_cast<unsigned>(p1);
    ctr[0] = hi1 ^ ctr[1] ^ key[0];
    ctr[1] = lo1;
    ctr[2] = hi0 ^ ctr[3] ^ key[1];
    ctr[3] = lo0;
    key[0] += 0x9E3779B9u;
    key[1] += 0xBB67AE85u;
}

// Philox-4x32-10 of counter (token, draw, 0, 0) under key (seed_lo, seed_hi); first word.
__device__ __forceinline__ unsigned philox_word(unsigned token, unsigned draw, unsigned seed_lo, unsigned seed_hi) {
    unsigned ctr[4] = {token, draw, 0u, 0u};
    unsigned key[2] = {seed_lo, seed_hi};
#pragma unroll
    for (int round = 0; round < 10; ++round) philox_round(ctr, key);
    return ctr[0];
}

__device__ __forceinline__ float gumbel_noise(unsigned word) {
    const float u = (static_cast<float>(word >> 8) + 0.5f) * (1.0f / 16777216.0f);
    return -logf(-logf(u));
}

struct ArgMax {
    float value;
    int index;
};

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    if (b.index < 0) return a;
    if (a.index < 0) return b;
    if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
    return a;
}

// Largest value, lowest index among equals.  All threads get the result.
__device__ ArgMax block_argmax(ArgMax mine, ArgMax* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        ArgMax other;
        other.value = __shfl_xor_sync(0xffffffffu, mine.value, offset);
        other.index = __shfl_xor_sync(0xffffffffu, mine.index, offset);
        mine = better(mine, other);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = mine;
    __syncthreads();
    if (warp == 0) {
        ArgMax w = lane < warps ? scratch[lane] : ArgMax{-INFINITY, -1};
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            ArgMax other;
            other.value = __shfl_xor_sync(0xffffffffu, w.value, offset);
            other.index = __shfl_xor_sync(0xffffffffu, w.index, offset);
            w = better(w, other);
        }
        if (lane == 0) scratch[32] = w;
    }
    __syncthreads();
    return scratch[32];
}

// Keeps, among the entries of work[] whose key equals `key`, the first `quota` by index and
// sets the others to -inf.
__device__ void keep_first_ties(float* work, int vocab, unsigned key, int quota, int* int_scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    int running = 0;
    for (int base = 0; base < vocab; base += blockDim.x) {
        const int v = base + threadIdx.x;
        const bool tie = v < vocab && order_key(work[v]) == key;
        const unsigned ballot = __ballot_sync(0xffffffffu, tie);
        const int before_in_warp = __popc(ballot & ((1u << lane) - 1u));
        __syncthreads();
        if (lane == 0) int_scratch[warp] = __popc(ballot);
        __syncthreads();
        int before = running;
        for (int w = 0; w < warp; ++w) before += int_scratch[w];
        int total = 0;
        for (int w = 0; w < warps; ++w) total += int_scratch[w];
        if (tie && before + before_in_warp >= quota) work[v] = -INFINITY;
        running += total;
    }
    __syncthreads();
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, float* __restrict__ work_all, const int* __restrict__ counts,
              const RowParams* __restrict__ params, int* __restrict__ out_tokens, int vocab) {
    __shared__ float hist_mass[256];
    __shared__ int hist_count[256];
    __shared__ ArgMax arg_scratch[33];
    __shared__ float float_scratch[33];
    __shared__ int int_scratch[32];
    __shared__ unsigned shared_prefix;
    __shared__ int shared_int;
    __shared__ float shared_float;

    const int row = blockIdx.x, tid = threadIdx.x;
    const RowParams p = params[row];
    const float* src = logits + static_cast<size_t>(row) * vocab;
    float* work = work_all + static_cast<size_t>(row) * vocab;
    const int* row_counts = (counts != nullptr && p.count_slot >= 0) ? counts + static_cast<size_t>(p.count_slot) * vocab : nullptr;
    const bool greedy = p.temperature == 0.0f;
    const bool scale = p.temperature > 0.0f;

    // Ban, penalties, temperature; running arg-max.
    ArgMax best{-INFINITY, -1};
    for (int v = tid; v < vocab; v += blockDim.x) {
        float x = src[v];
#pragma unroll
        for (int b = 0; b < kMaxBanned; ++b) x = (p.banned[b] == v) ? -INFINITY : x;
        const int count = row_counts ? row_counts[v] : 0;
        if (count > 0) {
            if (p.repetition_penalty != 1.0f) x = x > 0.0f ? x / p.repetition_penalty : x * p.repetition_penalty;
            x -= p.presence_penalty;
        }
        x -= p.frequency_penalty * static_cast<float>(count);
        if (scale) x = x / p.temperature;
        work[v] = x;
        if (x == x) best = better(best, ArgMax{x, v});
    }
    best = block_argmax(best, arg_scratch);
    if (greedy || best.index < 0) {
        if (tid == 0) out_tokens[row] = best.index < 0 ? 0 : best.index;
        return;
    }
    const float row_max = best.value;

    // top-k: the k-th largest key, then ties by index.
    if (p.top_k > 0 && p.top_k < vocab) {
        unsigned prefix = 0;
        int remaining = p.top_k;   // rank (1-based, from the top) looked for inside the current prefix
        int equal = 0;
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
            if (tid < 256) hist_count[tid] = 0;
            __syncthreads();
            for (int v = tid; v < vocab; v += blockDim.x) {
                const unsigned key = order_key(work[v]);
                if ((key & mask) == prefix) atomicAdd(&hist_count[(key >> shift) & 0xffu], 1);
            }
            __syncthreads();
            if (tid == 0) {
                int seen = 0, bin = 255;
                for (; bin > 0; --bin) {
                    if (seen + hist_count[bin] >= remaining) break;
                    seen += hist_count[bin];
                }
                shared_prefix = prefix | (static_cast<unsigned>(bin) << shift);
                shared_int = remaining - seen;
                int_scratch[0] = hist_count[bin];
            }
            __syncthreads();
            prefix = shared_prefix;
            remaining = shared_int;
            equal = int_scratch[0];
            __syncthreads();
        }
        // prefix = key of the k-th largest; `remaining` of the `equal` entries with that key stay.
        for (int v = tid; v < vocab; v += blockDim.x)
            if (order_key(work[v]) < prefix) work[v] = -INFINITY;
        __syncthreads();
        if (remaining < equal) keep_first_ties(work, vocab, prefix, remaining, int_scratch);
    }

    // top-p: drop tokens whose preceding cumulative probability (descending order) >= p.
    if (p.top_p < 1.0f) {
        float local = 0.0f;
        for (int v = tid; v < vocab; v += blockDim.x) local += expf(work[v] - row_max);
        const float total = block_sum(local, float_scratch);
        const float limit = p.top_p * total;
        unsigned prefix = 0;
        float before = 0.0f;   // mass of everything above the current prefix
        int equal = 0;
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
            if (tid < 256) {
                hist_mass[tid] = 0.0f;
                hist_count[tid] = 0;
            }
            __syncthreads();
            for (int v = tid; v < vocab; v += blockDim.x) {
                const float x = work[v];
                const unsigned key = order_key(x);
                if ((key & mask) == prefix && x > -INFINITY) {
                    atomicAdd(&hist_mass[(key >> shift) & 0xffu], expf(x - row_max));
                    atomicAdd(&hist_count[(key >> shift) & 0xffu], 1);
                }
            }
            __syncthreads();
            if (tid == 0) {
                // The lowest non-empty bin whose preceding mass is still below the limit.
                float cumulative = before;
                int chosen = -1;
                float chosen_before = before;
                for (int bin = 255; bin >= 0; --bin) {
                    if (hist_count[bin] == 0) continue;
                    if (cumulative < limit || chosen < 0) {
                        chosen = bin;
                        chosen_before = cumulative;
                    } else {
                        break;
                    }
                    cumulative += hist_mass[bin];
                }
                shared_prefix = prefix | (static_cast<unsigned>(chosen < 0 ? 0 : chosen) << shift);
                shared_float = chosen_before;
                shared_int = chosen < 0 ? 0 : hist_count[chosen];
            }
            __syncthreads();
            prefix = shared_prefix;
            before = shared_float;
            equal = shared_int;
            __syncthreads();
        }
        // Entries with key `prefix` are equal; rank r among them stays iff before + r * mass < limit.
        float tie_value = -INFINITY;
        for (int v = tid; v < vocab; v += blockDim.x) {
            const float x = work[v];
            const unsigned key = order_key(x);
            if (key < prefix) work[v] = -INFINITY;
            if (key == prefix) tie_value = x;
        }
        __syncthreads();
        if (equal > 1) {
            // All threads need the tie value: reduce it.
            const float value = block_max(tie_value, float_scratch);
            const float mass = expf(value - row_max);
            int quota = 1;
            while (quota < equal && before + static_cast<float>(quota) * mass < limit) ++quota;
            if (quota < equal) keep_first_ties(work, vocab, prefix, quota, int_scratch);
        }
    }

    // min-p and the draw: arg-max of logit + Gumbel noise over what is left.
    const float cutoff = p.min_p > 0.0f ? row_max + logf(p.min_p) : -INFINITY;
    ArgMax pick{-INFINITY, -1};
    for (int v = tid; v < vocab; v += blockDim.x) {
        const float x = work[v];
        if (x > -INFINITY && x >= cutoff) {
            const float g = gumbel_noise(philox_word(static_cast<unsigned>(v), p.draw, p.seed_lo, p.seed_hi));
            pick = better(pick, ArgMax{x + g, v});
        } else if (x > -INFINITY) {
            work[v] = -INFINITY;   // work[] ends up holding the fully processed logits
        }
    }
    pick = block_argmax(pick, arg_scratch);
    if (tid == 0) out_tokens[row] = pick.index < 0 ? best.index : pick.index;
}

// Greedy fast path: the arg-max of each row, no scratch.
__global__ void __launch_bounds__(kSampleThreads)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out_tokens, int vocab) {
    __shared__ ArgMax arg_scratch[33];
    const float* src = logits + static_cast<size_t>(blockIdx.x) * vocab;
    ArgMax best{-INFINITY, -1};
    for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
        const float x = src[v];
        if (x == x) best = better(best, ArgMax{x, v});
    }
    best = block_argmax(best, arg_scratch);
    if (threadIdx.x == 0) out_tokens[blockIdx.x] = best.index < 0 ? 0 : best.index;
}

// Greedy in two steps for rows too long for one block to scan quickly: each block of grid (rows, chunks)
// finds the best of its chunk, then one warp per row picks among the chunks' bests (lowest index wins ties,
// chunks being in index order).
__global__ void __launch_bounds__(256)
argmax_chunk_kernel(const float* __restrict__ logits, float* __restrict__ chunk_values, int* __restrict__ chunk_indices, int vocab, int chunk) {
    __shared__ ArgMax arg_scratch[33];
    const int row = blockIdx.x, part = blockIdx.y;
    const float* src = logits + static_cast<size_t>(row) * vocab;
    const int begin = part * chunk, end = min(vocab, begin + chunk);
    ArgMax best{-INFINITY, -1};
    for (int v = begin + threadIdx.x; v < end; v += blockDim.x) {
        const float x = src[v];
        if (x == x) best = better(best, ArgMax{x, v});
    }
    best = block_argmax(best, arg_scratch);
    if (threadIdx.x == 0) {
        chunk_values[row * gridDim.y + part] = best.value;
        chunk_indices[row * gridDim.y + part] = best.index;
    }
}

__global__ void argmax_merge_kernel(const float* __restrict__ chunk_values, const int* __restrict__ chunk_indices, int* __restrict__ out_tokens, int chunks) {
    const int row = blockIdx.x;
    ArgMax best{-INFINITY, -1};
    for (int part = threadIdx.x; part < chunks; part += 32) best = better(best, ArgMax{chunk_values[row * chunks + part], chunk_indices[row * chunks + part]});
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        ArgMax other;
        other.value = __shfl_xor_sync(0xffffffffu, best.value, offset);
        other.index = __shfl_xor_sync(0xffffffffu, best.index, offset);
        best = better(best, other);
    }
    if (threadIdx.x == 0) out_tokens[row] = best.index < 0 ? 0 : best.index;
}

// counts[slot, add[i]] += 1 and counts[slot, remove[i]] -= 1 (negative ids are skipped).
__global__ void update_counts_kernel(int* counts, const int* slots, const int* add, const int* remove, int rows, int vocab) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows || slots[i] < 0) return;
    int* row = counts + static_cast<size_t>(slots[i]) * vocab;
    if (add[i] >= 0 && add[i] < vocab) atomicAdd(&row[add[i]], 1);
    if (remove[i] >= 0 && remove[i] < vocab) atomicAdd(&row[remove[i]], -1);
}

}  // namespace lb

extern "C" {

int lb_sample_params_size() { return static_cast<int>(sizeof(lb::RowParams)); }

int lb_sample(const float* logits, float* work, const int* counts, const void* params, int* out_tokens, int rows,
              int vocab, cudaStream_t stream) {
    if (rows == 0) return 0;
    lb::sample_kernel<<<rows, lb::kSampleThreads, 0, stream>>>(logits, work, counts, static_cast<const lb::RowParams*>(params),
                                                              out_tokens, vocab);
    return LB_LAUNCH_RESULT();
}

int lb_argmax(const float* logits, int* out_tokens, int rows, int vocab, cudaStream_t stream) {
    if (rows == 0) return 0;
    lb::argmax_kernel<<<rows, lb::kSampleThreads, 0, stream>>>(logits, out_tokens, vocab);
    return LB_LAUNCH_RESULT();
}

// scratch: rows * chunks floats followed by rows * chunks ints.
int lb_argmax_chunked(const float* logits, void* scratch, int* out_tokens, int rows, int vocab, int chunks, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (chunks < 1 || chunks > 1024) return -2;
    const int chunk = (vocab + chunks - 1) / chunks;
    float* values = static_cast<float*>(scratch);
    int* indices = reinterpret_cast<int*>(values + static_cast<size_t>(rows) * chunks);
    lb::argmax_chunk_kernel<<<dim3(rows, chunks), 256, 0, stream>>>(logits, values, indices, vocab, chunk);
    lb::argmax_merge_kernel<<<rows, 32, 0, stream>>>(values, indices, out_tokens, chunks);
    return LB_LAUNCH_RESULT();
}

int lb_update_counts(int* counts, const int* slots, const int* add, const int* remove, int rows, int vocab,
                     cudaStream_t stream) {
    if (rows == 0) return 0;
    lb::update_counts_kernel<<<(rows + 127) / 128, 128, 0, stream>>>(counts, slots, add, remove, rows, vocab);
    return LB_LAUNCH_RESULT();
}

}  // extern "C"
