// Embedding gather, RMS norm (with the residual sum fused in) and the gated activation.
//
// The residual stream is kept in 32-bit whatever the activation type is; the sum
// `residual + delta` and all norm statistics are computed in 32-bit.
#include "common.cuh"

namespace lb {

// residual[t, :] = float(table[ids[t], :]) * scale
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                             int dim, int vocab, float scale, int* status) {
    const int token = blockIdx.x;
    int id = ids[token];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) report_error(status, kBadToken);
        id = 0;
    }
    const T* row = table + static_cast<size_t>(id) * dim;
    float* dst = out + static_cast<size_t>(token) * dim;
    if (sizeof(T) == 2 && dim % 8 == 0) {
        // eight elements per thread and turn: one 16-byte load, two 16-byte stores
        for (int d = 8 * threadIdx.x; d < dim; d += 8 * blockDim.x) {
            const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(row) + d);
            const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
            const float2 a = __bfloat1622float2(pairs[0]), b = __bfloat1622float2(pairs[1]), c = __bfloat1622float2(pairs[2]), e = __bfloat1622float2(pairs[3]);
            *reinterpret_cast<float4*>(dst + d) = make_float4(a.x * scale, a.y * scale, b.x * scale, b.y * scale);
            *reinterpret_cast<float4*>(dst + d + 4) = make_float4(c.x * scale, c.y * scale, e.x * scale, e.y * scale);
        }
        return;
    }
    for (int d = threadIdx.x; d < dim; d += blockDim.x) dst[d] = to_float(row[d]) * scale;
}

// One block per output row r.  src = rows ? rows[r] : r.
//   h = x[src] (+ delta[src]);   if write_back: x[src] = h  (x is the 32-bit residual stream)
//   n = T(h * rsqrt(mean(h^2) + eps));   out[r] = T(n * T(w + offset))
// The two roundings to T follow the reference's norm in its "only normalisation is upcast" mode.
// With `slices` > 0 the delta is a product left as its K slices' partial sums: `partials[s][src][d]`, `slice_stride`
// floats apart, added in slice order and rounded to T as the product's own epilogue would have stored it.
template <typename TX, typename T>
__global__ void rmsnorm_kernel(TX* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ partials, int slices,
                               size_t slice_stride, const float* __restrict__ weight,
                               const int* __restrict__ rows, T* __restrict__ out, int dim, float eps,
                               float scale_offset, int write_back) {
    extern __shared__ float shared[];
    // Launched to start early: it is resident when the kernel before it ends (no launch in between).  Only then
    // may the product after it start and pull its weights towards L2: under the stream of the kernel before,
    // those weights would be gone again before they are read.
    wait_for_previous_kernel();
    allow_next_kernel();
    float* row_cache = shared;           // dim floats
    float* scratch = shared + dim;       // 33 floats
    const int r = blockIdx.x;
    const size_t src = rows ? static_cast<size_t>(rows[r]) : static_cast<size_t>(r);
    TX* xr = x + src * dim;
    const T* dr = delta ? delta + src * dim : nullptr;
    const float* pr = slices > 0 ? partials + src * dim : nullptr;
    const bool adds = dr != nullptr || pr != nullptr;
    float sum = 0.0f;
    constexpr bool kVector = sizeof(TX) == 4 && sizeof(T) == 2;   // 32-bit stream in, bfloat16 out: four elements at a time
    if (kVector && dim % 4 == 0) {
        for (int d = 4 * threadIdx.x; d < dim; d += 4 * blockDim.x) {
            float4 h = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(xr) + d);
            if (dr) {
                const uint2 raw = *reinterpret_cast<const uint2*>(dr + d);
                const float2 low = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                const float2 high = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                h.x += low.x;
                h.y += low.y;
                h.z += high.x;
                h.w += high.y;
            }
            if (pr) {
                // Four slices' loads leave before the first is added (the order of the additions stays).
                float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                int s = 0;
                for (; s + 4 <= slices; s += 4) {
                    float4 part[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) part[u] = __ldcs(reinterpret_cast<const float4*>(pr + static_cast<size_t>(s + u) * slice_stride + d));
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        total.x += part[u].x;
                        total.y += part[u].y;
                        total.z += part[u].z;
                        total.w += part[u].w;
                    }
                }
                for (; s < slices; ++s) {
                    const float4 part = __ldcs(reinterpret_cast<const float4*>(pr + static_cast<size_t>(s) * slice_stride + d));
                    total.x += part.x;
                    total.y += part.y;
                    total.z += part.z;
                    total.w += part.w;
                }
                h.x += round_to<T>(total.x);
                h.y += round_to<T>(total.y);
                h.z += round_to<T>(total.z);
                h.w += round_to<T>(total.w);
            }
            *reinterpret_cast<float4*>(row_cache + d) = h;
            sum += h.x * h.x + h.y * h.y + h.z * h.z + h.w * h.w;
        }
    } else {
        for (int d = threadIdx.x; d < dim; d += blockDim.x) {
            float h = to_float(xr[d]);
            if (dr) h += to_float(dr[d]);
            if (pr) {
                float total = 0.0f;
                for (int s = 0; s < slices; ++s) total += pr[static_cast<size_t>(s) * slice_stride + d];
                h += round_to<T>(total);
            }
            row_cache[d] = h;
            sum += h * h;
        }
    }
    const float total = block_sum(sum, scratch);
    const float inv = rsqrtf(total / static_cast<float>(dim) + eps);
    T* dst = out + static_cast<size_t>(r) * dim;
    if (kVector && dim % 4 == 0) {
        for (int d = 4 * threadIdx.x; d < dim; d += 4 * blockDim.x) {
            const float4 h = *reinterpret_cast<const float4*>(row_cache + d);
            if (write_back && adds) *reinterpret_cast<float4*>(reinterpret_cast<float*>(xr) + d) = h;
            const float4 w = *reinterpret_cast<const float4*>(weight + d);
            const __nv_bfloat162 low = __floats2bfloat162_rn(round_to<T>(h.x * inv) * round_to<T>(w.x + scale_offset),
                                                             round_to<T>(h.y * inv) * round_to<T>(w.y + scale_offset));
            const __nv_bfloat162 high = __floats2bfloat162_rn(round_to<T>(h.z * inv) * round_to<T>(w.z + scale_offset),
                                                              round_to<T>(h.w * inv) * round_to<T>(w.w + scale_offset));
            uint2 packed;
            packed.x = *reinterpret_cast<const uint32_t*>(&low);
            packed.y = *reinterpret_cast<const uint32_t*>(&high);
            *reinterpret_cast<uint2*>(dst + d) = packed;
        }
    } else {
        for (int d = threadIdx.x; d < dim; d += blockDim.x) {
            const float h = row_cache[d];
            if (write_back && adds) xr[d] = from_float<TX>(h);
            const float n = round_to<T>(h * inv);
            const float w = round_to<T>(weight[d] + scale_offset);
            dst[d] = from_float<T>(n * w);
        }
    }
}

// x += delta on the 32-bit residual stream (used by norms that have no fused form).
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ x, const T* __restrict__ delta, size_t count) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) x[i] += to_float(delta[i]);
}

// out[r, :] = src[rows[r], :]
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, const int* __restrict__ rows, T* __restrict__ out, int dim) {
    const size_t from = static_cast<size_t>(rows[blockIdx.x]) * dim, to = static_cast<size_t>(blockIdx.x) * dim;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) out[to + d] = src[from + d];
}

__device__ __forceinline__ float activate(float v, int activation) {
    if (activation == 0) return v / (1.0f + expf(-v));                                   // silu
    if (activation == 1) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));    // gelu (exact)
    return v;                                                                            // identity
}

// fused[t] = [up (hidden) ; gate (hidden)];  out[t, f] = T(up * act(gate)), 32-bit inside.
template <typename T>
__global__ void gated_activation_kernel(const T* __restrict__ fused, T* __restrict__ out, int hidden, size_t count,
                                        int activation) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const size_t token = i / hidden;
    const int f = static_cast<int>(i - token * hidden);
    const T* row = fused + token * 2 * static_cast<size_t>(hidden);
    const float up = to_float(row[f]);
    const float gate = to_float(row[hidden + f]);
    out[i] = from_float<T>(up * round_to<T>(activate(gate, activation)));
}

// The same, eight elements per thread with 16-byte accesses (hidden % 8 == 0).
__global__ void gated_activation_bf16x8_kernel(const __nv_bfloat16* __restrict__ fused, __nv_bfloat16* __restrict__ out, int hidden,
                                               size_t groups, int activation) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= groups) return;
    const int per_row = hidden / 8;
    const size_t token = i / per_row;
    const int f = static_cast<int>(i - token * per_row) * 8;
    const __nv_bfloat16* row = fused + token * 2 * static_cast<size_t>(hidden);
    const uint4 up_raw = *reinterpret_cast<const uint4*>(row + f);
    const uint4 gate_raw = *reinterpret_cast<const uint4*>(row + hidden + f);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&up_raw);
    const __nv_bfloat162* gate = reinterpret_cast<const __nv_bfloat162*>(&gate_raw);
    uint4 result_raw;
    __nv_bfloat162* result = reinterpret_cast<__nv_bfloat162*>(&result_raw);
#pragma unroll
    for (int pair = 0; pair < 4; ++pair) {
        const float2 u = __bfloat1622float2(up[pair]), g = __bfloat1622float2(gate[pair]);
        result[pair] = __floats2bfloat162_rn(u.x * round_to<__nv_bfloat16>(activate(g.x, activation)),
                                             u.y * round_to<__nv_bfloat16>(activate(g.y, activation)));
    }
    *reinterpret_cast<uint4*>(out + token * static_cast<size_t>(hidden) + f) = result_raw;
}

// Fills one slot of every per-request state with a 32-bit pattern (zero at admission).  `table`
// holds, per state tensor, its base address and the bytes one slot takes; block (x, y) fills a
// piece of state y's slot.  States whose slots are 16-byte multiples are written 16 bytes at a time.
__global__ void fill_slots_kernel(const long long* __restrict__ table, int slot, unsigned pattern) {
    const long long base = table[2 * blockIdx.y], bytes = table[2 * blockIdx.y + 1];
    unsigned char* begin = reinterpret_cast<unsigned char*>(base) + static_cast<size_t>(slot) * bytes;
    const size_t first = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x);
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    if ((bytes % 16 == 0) && (base % 16 == 0)) {
        const uint4 value = make_uint4(pattern, pattern, pattern, pattern);
        for (size_t i = first; i < static_cast<size_t>(bytes) / 16; i += stride) reinterpret_cast<uint4*>(begin)[i] = value;
    } else {
        // odd sizes: byte by byte, the pattern's bytes in address order
        for (size_t i = first; i < static_cast<size_t>(bytes); i += stride) {
            const size_t address = reinterpret_cast<size_t>(begin) + i;
            begin[i] = static_cast<unsigned char>(pattern >> (8 * (address & 3)));
        }
    }
}

// Token ids that were sampled on the device in the step before and have not been to the host: the last
// token of segment s is taken from row source[s] of `sampled` (source[s] < 0: the host wrote it).
__global__ void feed_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ segment_start, const int* __restrict__ segment_length,
                                   const int* __restrict__ source, const int* __restrict__ sampled, int sampled_rows, int segments, int* status) {
    const int segment = blockIdx.x * blockDim.x + threadIdx.x;
    if (segment >= segments) return;
    const int row = source[segment];
    if (row < 0) return;
    if (row >= sampled_rows) {
        report_error(status, kBadToken);
        return;
    }
    token_ids[segment_start[segment] + segment_length[segment] - 1] = sampled[row];
}

}  // namespace lb

extern "C" {

int lb_feed_tokens(int* token_ids, const int* segment_start, const int* segment_length, const int* source, const int* sampled, int sampled_rows,
                   int segments, int* status, cudaStream_t stream) {
    if (segments == 0) return 0;
    lb::feed_tokens_kernel<<<(segments + 127) / 128, 128, 0, stream>>>(token_ids, segment_start, segment_length, source, sampled, sampled_rows, segments, status);
    return LB_LAUNCH_RESULT();
}

// table: device array of `states` records (base address, bytes per slot), int64 each.
int lb_fill_slots(const long long* table, int states, long long largest_bytes, int slot, unsigned pattern, cudaStream_t stream) {
    if (states == 0 || largest_bytes == 0) return 0;
    long long pieces = (largest_bytes / 16 + 255) / 256;
    if (pieces < 1) pieces = 1;
    if (pieces > 64) pieces = 64;
    lb::fill_slots_kernel<<<dim3(static_cast<unsigned>(pieces), static_cast<unsigned>(states)), 256, 0, stream>>>(table, slot, pattern);
    return LB_LAUNCH_RESULT();
}

int lb_embed(const void* table, const int* ids, float* out, int tokens, int dim, int vocab, float scale, int dtype,
             int* status, cudaStream_t stream) {
    if (tokens == 0) return 0;
    LB_DISPATCH_DTYPE(dtype, {
        lb::embed_kernel<T><<<tokens, 256, 0, stream>>>(static_cast<const T*>(table), ids, out, dim, vocab, scale, status);
    })
    return LB_LAUNCH_RESULT();
}

// x_is_float: 1 when x is the 32-bit residual stream, 0 when x has the activation type.
// partials, slices, slice_stride: see rmsnorm_kernel (slices == 0: none); the vector path needs slice_stride % 4 == 0.
int lb_rmsnorm(void* x, int x_is_float, const void* delta, const float* partials, int slices, long long slice_stride, const float* weight,
               const int* rows, void* out, int out_rows, int dim, float eps, float scale_offset, int write_back, int dtype, cudaStream_t stream) {
    if (out_rows == 0) return 0;
    if (slices < 0 || (slices > 0 && (partials == nullptr || slice_stride < 0 || (dim % 4 == 0 && slice_stride % 4 != 0)))) return -2;
    const size_t shared = (static_cast<size_t>(dim) + 33) * sizeof(float);
    if (shared > 200 * 1024) return -2;
    // Few rows (decoding): the kernel is one trip to memory long if every thread has one piece of
    // the row, so a thread per four elements; many rows: 256 threads keep more rows resident per SM.
    int threads = dim >= 1024 ? 256 : 128;
    if (out_rows <= 64) {
        threads = ((dim + 3) / 4 + 31) / 32 * 32;
        threads = threads < 128 ? 128 : (threads > 1024 ? 1024 : threads);
    }
    LB_DISPATCH_DTYPE(dtype, {
        if (x_is_float) {
            auto kernel = lb::rmsnorm_kernel<float, T>;
            if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
            lb::launch_overlapped(kernel, dim3(out_rows), dim3(threads), shared, stream, static_cast<float*>(x), static_cast<const T*>(delta), partials, slices,
                                  static_cast<size_t>(slice_stride), weight, rows, static_cast<T*>(out), dim, eps, scale_offset, write_back);
        } else {
            auto kernel = lb::rmsnorm_kernel<T, T>;
            if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
            lb::launch_overlapped(kernel, dim3(out_rows), dim3(threads), shared, stream, static_cast<T*>(x), static_cast<const T*>(delta), partials, slices,
                                  static_cast<size_t>(slice_stride), weight, rows, static_cast<T*>(out), dim, eps, scale_offset, write_back);
        }
    })
    return LB_LAUNCH_RESULT();
}

int lb_residual_add(float* x, const void* delta, long long count, int dtype, cudaStream_t stream) {
    if (count == 0) return 0;
    const unsigned blocks = static_cast<unsigned>((count + 255) / 256);
    LB_DISPATCH_DTYPE(dtype, {
        lb::residual_add_kernel<T><<<blocks, 256, 0, stream>>>(x, static_cast<const T*>(delta), static_cast<size_t>(count));
    })
    return LB_LAUNCH_RESULT();
}

// element_size: 2 or 4 bytes per element (rows are copied bit for bit).
int lb_gather_rows(const void* src, const int* rows, void* out, int out_rows, int dim, int element_size,
                   cudaStream_t stream) {
    if (out_rows == 0) return 0;
    if (element_size == 4) {
        lb::gather_rows_kernel<float><<<out_rows, 256, 0, stream>>>(static_cast<const float*>(src), rows, static_cast<float*>(out), dim);
    } else if (element_size == 2) {
        lb::gather_rows_kernel<__nv_bfloat16><<<out_rows, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), rows,
                                                                           static_cast<__nv_bfloat16*>(out), dim);
    } else {
        return -1;
    }
    return LB_LAUNCH_RESULT();
}

int lb_gated_activation(const void* fused, void* out, int tokens, int hidden, int activation, int dtype,
                        cudaStream_t stream) {
    const size_t count = static_cast<size_t>(tokens) * hidden;
    if (count == 0) return 0;
    if (dtype == lb::kBFloat16 && hidden % 8 == 0) {
        const size_t groups = count / 8;
        lb::gated_activation_bf16x8_kernel<<<static_cast<unsigned>((groups + 255) / 256), 256, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(fused), static_cast<__nv_bfloat16*>(out), hidden, groups, activation);
        return LB_LAUNCH_RESULT();
    }
    const unsigned blocks = static_cast<unsigned>((count + 255) / 256);
    LB_DISPATCH_DTYPE(dtype, {
        lb::gated_activation_kernel<T><<<blocks, 256, 0, stream>>>(static_cast<const T*>(fused), static_cast<T*>(out), hidden, count, activation);
    })
    return LB_LAUNCH_RESULT();
}

}  // extern "C"
