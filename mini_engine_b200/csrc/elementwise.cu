// Memory-bound kernels between the matrix products: embedding lookup (plain, and with a second
// table chosen by the pair of the previous and the current token), residual sum fused with RMSNorm,
// the SwiGLU gate on partial sums, and q/k norm (per head, or over whole projections) + rotary +
// cache write.  Statistics, angles and sums are 32-bit; outputs are rounded once.
//
// Formulas restate YuvGev00/mini-engine: src/mini_engine/model.py:59-69 (RMSNorm),
// :72-90 (rotary, rotate-half), :113-116 (norm before rotation, v untouched), :130 (SwiGLU),
// src/mini_engine/attention.py:118-121 (new K/V go to their slots before attention reads).
#include "common.cuh"

#include <algorithm>

// ------------------------------------------------------------------------------ embedding

// One block per token.  VEC: the width is a multiple of 8 and both pointers are 16-byte aligned;
// a thread then moves eight elements per step.
template <typename T, bool VEC>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int hidden, int vocab, float multiplier) {
    const int token = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    const int id = ids[token];
    float* row_out = out + static_cast<size_t>(token) * hidden;
    if (id < 0 || id >= vocab) {  // the host validates ids; never read outside the table
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) row_out[i] = 0.0f;
        return;
    }
    const T* row = table + static_cast<size_t>(id) * hidden;
    if (VEC) {
        for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
            float v[8];
            if (sizeof(T) == 2) {
                const uint4 raw = *reinterpret_cast<const uint4*>(row + i);
                const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(pairs[j]);
                    v[2 * j] = f.x, v[2 * j + 1] = f.y;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = to_float(row[i + j]);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] *= multiplier;  // 1 for a model without embedding scaling: exact
            *reinterpret_cast<float4*>(row_out + i) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(row_out + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) row_out[i] = to_float(row[i]) * multiplier;
    }
}

// out[t][:] = table[ids[t]][:] * multiplier, widened to float32.
ME_EXPORT int me_embedding(const void* table, int table_type, const int* ids, float* out, int tokens,
                           int hidden, int vocab, float multiplier, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const bool vec = hidden % 8 == 0 && reinterpret_cast<uintptr_t>(table) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
    const int threads = vec ? std::min(512, std::max(32, (hidden / 8 + 31) / 32 * 32)) : (hidden >= 1024 ? 256 : 128);
    if (table_type == ME_BF16) {
        const auto* t = static_cast<const __nv_bfloat16*>(table);
        return vec ? launch_kernel(embedding_kernel<__nv_bfloat16, true>, tokens, threads, 0, stream, t, ids, out, hidden, vocab, multiplier)
                   : launch_kernel(embedding_kernel<__nv_bfloat16, false>, tokens, threads, 0, stream, t, ids, out, hidden, vocab, multiplier);
    }
    const auto* t = static_cast<const float*>(table);
    return vec ? launch_kernel(embedding_kernel<float, true>, tokens, threads, 0, stream, t, ids, out, hidden, vocab, multiplier)
               : launch_kernel(embedding_kernel<float, false>, tokens, threads, 0, stream, t, ids, out, hidden, vocab, multiplier);
}

// ------------------------------------------------------------- what a head may do to logits

// logits[r][v] = cap(logits[r][v] * scale + bias[v]) with cap(y) = soft_cap * tanh(y / soft_cap) when
// soft_cap > 0, in place; `bias` may be null.  For heads that have a bias, a logit scale or a
// soft cap; a plain head never launches this.
__global__ void logits_finish_kernel(float* __restrict__ logits, const float* __restrict__ bias, float scale,
                                     float soft_cap, int vocab) {
    pdl_trigger();
    pdl_wait();
    float* row = logits + static_cast<size_t>(blockIdx.y) * vocab;
    for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < vocab; v += gridDim.x * blockDim.x) {
        float y = row[v] * scale;
        if (bias != nullptr) y += bias[v];
        if (soft_cap > 0.0f) y = soft_cap * tanhf(y / soft_cap);
        row[v] = y;
    }
}

ME_EXPORT int me_logits_finish(float* logits, const float* bias, float scale, float soft_cap, int rows, int vocab,
                               cudaStream_t stream) {
    if (rows <= 0 || vocab <= 0) return 0;
    if (rows > 65535) return ME_ERR_ARGUMENT;
    const int blocks = std::min((vocab + 255) / 256, 1024);
    return launch_kernel(logits_finish_kernel, dim3(blocks, rows), 256, 0, stream, logits, bias, scale, soft_cap, vocab);
}

// --------------------------------------------------------------- residual sum + RMSNorm

constexpr int MAX_UNROLLED_SPLITS = 8;

__device__ __forceinline__ void store4(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = packed;
}

// One block per output row.  x_row = x_scale * x[src] + sum_s pending[s][src] (ascending s); when
// `rows` is null the sum is written back to x (the residual stream advances), otherwise only
// the listed rows are read and x is left alone.  out = weight * x_row * rsqrt(mean(x_row^2) + eps).
// With `keep_normed` (and no `rows`) it is the normalised row, in float32, that is written back to x
// instead of the sum: a layer whose norm follows the sum.  x_scale is 1 in pre-norm layers (exact).
// VEC: hidden is a multiple of 4 and every pointer is 16-byte aligned; all loads of a thread are
// then issued before any of them is used, which is what matters when only a few rows run.
//
// The sum of squares is defined over LANES "lanes" (256, 512 or 1024, chosen from the width
// alone): lane v adds the squares of its columns 4v..4v+3 (+ 4 LANES j) in ascending order, the 32
// lanes of a warp are added by a butterfly, and the warps' sums in ascending order.  A block of
// THREADS = LANES threads has one lane per thread (every load of a short row in flight at once:
// few rows); a block of THREADS < LANES threads plays LANES / THREADS lanes per thread with one
// partial sum each, which gives the same bits with more blocks per SM (many rows).
template <typename OutT, bool VEC, int LANES, int THREADS>
__global__ void __launch_bounds__(THREADS)
add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ pending, int splits, size_t split_stride,
                   const float* __restrict__ weight, float eps, OutT* __restrict__ out,
                   const int* __restrict__ rows, int hidden, const float* __restrict__ pending_scale,
                   float x_scale, int keep_normed) {
    constexpr int PLAYED = LANES / THREADS;  // lanes per thread
    extern __shared__ float row_cache[];  // [hidden]
    __shared__ float warp_partial[LANES / 32];
    const int out_row = blockIdx.x;
    pdl_trigger();
    // The norm's weight and the step's row list do not come from the previous kernel: fetch them
    // ahead of the wait.
    const int src = rows ? rows[out_row] : out_row;
    float4 first_weight = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (VEC && threadIdx.x * 4 < hidden) first_weight = *reinterpret_cast<const float4*>(weight + threadIdx.x * 4);
    pdl_wait();
    float* x_row = x + static_cast<size_t>(src) * hidden;
    const float* pending_row = pending + static_cast<size_t>(src) * hidden;
    // keep_normed: the stream itself becomes the normalised row (a layer whose norm follows the sum).
    const bool write_back = !rows && splits > 0 && !keep_normed;
    const bool write_normed = !rows && keep_normed;
    float sum_sq[PLAYED];
#pragma unroll
    for (int k = 0; k < PLAYED; ++k) sum_sq[k] = 0.0f;
    if (VEC && splits <= MAX_UNROLLED_SPLITS) {
        for (int base = 0; base < hidden; base += LANES * 4) {
#pragma unroll
            for (int k = 0; k < PLAYED; ++k) {
                const int i = base + (k * THREADS + threadIdx.x) * 4;
                if (i >= hidden) continue;
                float4 v = *reinterpret_cast<const float4*>(x_row + i);
                v.x *= x_scale; v.y *= x_scale; v.z *= x_scale; v.w *= x_scale;  // 1 in a pre-norm layer: exact
                float4 part[MAX_UNROLLED_SPLITS];
#pragma unroll
                for (int s = 0; s < MAX_UNROLLED_SPLITS; ++s)
                    if (s < splits) part[s] = *reinterpret_cast<const float4*>(pending_row + s * split_stride + i);
                if (pending_scale != nullptr && splits > 0) {
                    // x + scale * (sum of the partial sums): the part's output is whole before it is scaled
                    float4 sum = part[0];
#pragma unroll
                    for (int s = 1; s < MAX_UNROLLED_SPLITS; ++s)
                        if (s < splits) { sum.x += part[s].x; sum.y += part[s].y; sum.z += part[s].z; sum.w += part[s].w; }
                    const float4 c = *reinterpret_cast<const float4*>(pending_scale + i);
                    v.x = fmaf(c.x, sum.x, v.x); v.y = fmaf(c.y, sum.y, v.y); v.z = fmaf(c.z, sum.z, v.z); v.w = fmaf(c.w, sum.w, v.w);
                } else {
#pragma unroll
                    for (int s = 0; s < MAX_UNROLLED_SPLITS; ++s)
                        if (s < splits) { v.x += part[s].x; v.y += part[s].y; v.z += part[s].z; v.w += part[s].w; }
                }
                *reinterpret_cast<float4*>(row_cache + i) = v;
                if (write_back) *reinterpret_cast<float4*>(x_row + i) = v;
                sum_sq[k] = fmaf(v.x, v.x, sum_sq[k]);
                sum_sq[k] = fmaf(v.y, v.y, sum_sq[k]);
                sum_sq[k] = fmaf(v.z, v.z, sum_sq[k]);
                sum_sq[k] = fmaf(v.w, v.w, sum_sq[k]);
            }
        }
    } else {
        for (int base = 0; base < hidden; base += LANES) {
#pragma unroll
            for (int k = 0; k < PLAYED; ++k) {
                const int i = base + k * THREADS + threadIdx.x;
                if (i >= hidden) continue;
                float v = x_row[i] * x_scale;
                if (pending_scale != nullptr && splits > 0) {
                    float sum = pending_row[i];
                    for (int s = 1; s < splits; ++s) sum += pending_row[s * split_stride + i];
                    v = fmaf(pending_scale[i], sum, v);
                } else {
                    for (int s = 0; s < splits; ++s) v += pending_row[s * split_stride + i];
                }
                row_cache[i] = v;
                if (write_back) x_row[i] = v;
                sum_sq[k] = fmaf(v, v, sum_sq[k]);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < PLAYED; ++k) {
        const float warp_total = warp_sum(sum_sq[k]);
        if ((threadIdx.x & 31) == 0) warp_partial[k * (THREADS / 32) + (threadIdx.x >> 5)] = warp_total;
    }
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < LANES / 32; ++w) total += warp_partial[w];
    const float inv = rsqrtf(total / static_cast<float>(hidden) + eps);
    OutT* out_ptr = out + static_cast<size_t>(out_row) * hidden;
    if (VEC) {
        for (int i = threadIdx.x * 4; i < hidden; i += THREADS * 4) {
            const float4 v = *reinterpret_cast<const float4*>(row_cache + i);
            const float4 w = i == threadIdx.x * 4 ? first_weight : *reinterpret_cast<const float4*>(weight + i);
            const float4 y = make_float4(w.x * (v.x * inv), w.y * (v.y * inv), w.z * (v.z * inv), w.w * (v.w * inv));
            store4(out_ptr + i, y);
            if (write_normed) *reinterpret_cast<float4*>(x_row + i) = y;
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += THREADS) {
            const float y = weight[i] * (row_cache[i] * inv);
            out_ptr[i] = from_float<OutT>(y);
            if (write_normed) x_row[i] = y;
        }
    }
}

template <typename OutT, bool VEC, int LANES, int THREADS>
static int launch_add_rmsnorm_threads(float* x, const float* pending, int splits, size_t split_stride,
                                      const float* weight, float eps, OutT* out, const int* rows, int count, int hidden,
                                      cudaStream_t stream, const float* pending_scale, float x_scale, int keep_normed) {
    const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
    auto kernel = add_rmsnorm_kernel<OutT, VEC, LANES, THREADS>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_kernel(kernel, count, THREADS, smem, stream, x, pending, splits, split_stride, weight, eps, out,
                         rows, hidden, pending_scale, x_scale, keep_normed);
}

// Few rows: one lane per thread.  Many rows: 256 threads per row, more rows per SM.  The lanes
// (hence the bits of the result) depend on the width alone.
constexpr int NORM_MANY_ROWS = 256;

template <typename OutT, bool VEC, int LANES>
static int launch_add_rmsnorm_lanes(float* x, const float* pending, int splits, size_t split_stride, const float* weight,
                                    float eps, OutT* out, const int* rows, int count, int hidden, cudaStream_t stream,
                                    const float* pending_scale, float x_scale, int keep_normed) {
    if (count >= NORM_MANY_ROWS)
        return launch_add_rmsnorm_threads<OutT, VEC, LANES, 256>(x, pending, splits, split_stride, weight, eps, out, rows, count, hidden, stream, pending_scale, x_scale, keep_normed);
    return launch_add_rmsnorm_threads<OutT, VEC, LANES, LANES>(x, pending, splits, split_stride, weight, eps, out, rows, count, hidden, stream, pending_scale, x_scale, keep_normed);
}

template <typename OutT, bool VEC>
static int launch_add_rmsnorm(float* x, const float* pending, int splits, size_t split_stride, const float* weight,
                              float eps, OutT* out, const int* rows, int count, int hidden, cudaStream_t stream,
                                    const float* pending_scale, float x_scale, int keep_normed) {
    if (VEC && hidden > 2048)
        return launch_add_rmsnorm_lanes<OutT, VEC, 1024>(x, pending, splits, split_stride, weight, eps, out, rows, count, hidden, stream, pending_scale, x_scale, keep_normed);
    if (VEC && hidden > 1024)
        return launch_add_rmsnorm_lanes<OutT, VEC, 512>(x, pending, splits, split_stride, weight, eps, out, rows, count, hidden, stream, pending_scale, x_scale, keep_normed);
    return launch_add_rmsnorm_lanes<OutT, VEC, 256>(x, pending, splits, split_stride, weight, eps, out, rows, count, hidden, stream, pending_scale, x_scale, keep_normed);
}

static bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

ME_EXPORT int me_add_rmsnorm(float* x, const float* pending, int splits, long long split_stride,
                             const float* weight, float eps, void* out, int out_type, const int* rows,
                             int count, int hidden, const float* pending_scale, float x_scale, int keep_normed,
                             cudaStream_t stream) {
    if (count <= 0) return 0;
    if (static_cast<size_t>(hidden) * sizeof(float) > 200 * 1024) return ME_ERR_UNSUPPORTED;
    // Which path runs depends on the width and on the alignment of the engine's persistent
    // buffers only, never on the batch, so a row's statistics are the same bits in every step.
    const bool vec = hidden % 4 == 0 && aligned16(x) && aligned16(weight) && aligned16(out) &&
                     (pending == nullptr || (aligned16(pending) && split_stride % 4 == 0)) && aligned16(pending_scale);
    const size_t stride = static_cast<size_t>(split_stride);
    if (out_type == ME_BF16) {
        auto* o = static_cast<__nv_bfloat16*>(out);
        return vec ? launch_add_rmsnorm<__nv_bfloat16, true>(x, pending, splits, stride, weight, eps, o, rows, count, hidden, stream, pending_scale, x_scale, keep_normed)
                   : launch_add_rmsnorm<__nv_bfloat16, false>(x, pending, splits, stride, weight, eps, o, rows, count, hidden, stream, pending_scale, x_scale, keep_normed);
    }
    auto* o = static_cast<float*>(out);
    return vec ? launch_add_rmsnorm<float, true>(x, pending, splits, stride, weight, eps, o, rows, count, hidden, stream, pending_scale, x_scale, keep_normed)
               : launch_add_rmsnorm<float, false>(x, pending, splits, stride, weight, eps, o, rows, count, hidden, stream, pending_scale, x_scale, keep_normed);
}

// -------------------------------------------------------------- residual sum + layer norm

// One block per output row.  x_row = x[src] + add_bias + sum_s first[s][src] + sum_s second[s][src] (each sum in
// ascending s); when `rows` is null and something was added the sum is written back to x.  Then
// out = (x_row - mean) * rsqrt(var + eps) * weight + bias with var the mean of the squared deviations from the
// mean (two passes over the row, which stays in shared memory), all in float32.  `second` is the output of a
// second sublayer that read the same normalised input as the first (a parallel block); `add_bias` is the bias of
// the first sublayer's output projection.  Column i goes to the partial sum of thread i % 256 in ascending
// order, warps are added by a butterfly and then in ascending order: a row's statistics never depend on the batch.
struct LayerNormArgs {
    float* x;
    const float* first;
    int first_splits;
    size_t first_stride;
    const float* second;
    int second_splits;
    size_t second_stride;
    const float* add_bias;
    const float* weight;
    const float* bias;
    float eps;
    void* out;
    const int* rows;
    int hidden;
};

__device__ __forceinline__ float block_sum_256(float v, float* scratch) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += scratch[w];
    __syncthreads();
    return total;
}

template <typename OutT>
__global__ void __launch_bounds__(256) add_layernorm_kernel(LayerNormArgs a) {
    extern __shared__ float row_cache[];  // [hidden]
    __shared__ float scratch[8];
    const int out_row = blockIdx.x;
    pdl_trigger();
    const int src = a.rows ? a.rows[out_row] : out_row;
    pdl_wait();
    const size_t offset = static_cast<size_t>(src) * a.hidden;
    float* x_row = a.x + offset;
    const bool write_back = !a.rows && (a.first_splits > 0 || a.second_splits > 0 || a.add_bias != nullptr);
    float sum = 0.0f;
    for (int i = threadIdx.x; i < a.hidden; i += 256) {
        float v = x_row[i];
        if (a.first_splits > 0) {
            float part = a.first[offset + i];
            for (int s = 1; s < a.first_splits; ++s) part += a.first[s * a.first_stride + offset + i];
            if (a.add_bias) part += a.add_bias[i];
            v += part;
        } else if (a.add_bias) {
            v += a.add_bias[i];
        }
        if (a.second_splits > 0) {
            float part = a.second[offset + i];
            for (int s = 1; s < a.second_splits; ++s) part += a.second[s * a.second_stride + offset + i];
            v += part;
        }
        row_cache[i] = v;
        if (write_back) x_row[i] = v;
        sum += v;
    }
    const float mean = block_sum_256(sum, scratch) / static_cast<float>(a.hidden);
    float squares = 0.0f;
    for (int i = threadIdx.x; i < a.hidden; i += 256) {
        const float d = row_cache[i] - mean;
        squares = fmaf(d, d, squares);
    }
    const float inv = rsqrtf(block_sum_256(squares, scratch) / static_cast<float>(a.hidden) + a.eps);
    OutT* out_ptr = static_cast<OutT*>(a.out) + static_cast<size_t>(out_row) * a.hidden;
    for (int i = threadIdx.x; i < a.hidden; i += 256)
        out_ptr[i] = from_float<OutT>(fmaf((row_cache[i] - mean) * inv, a.weight[i], a.bias[i]));
}

// The same over LANES "lanes" of four consecutive columns each, as in add_rmsnorm_kernel: lane v holds columns
// 4v..4v+3 (+ 4 LANES j) and one partial sum; a warp's 32 lanes are added by a butterfly and the warps in ascending
// order.  LANES follows from the width alone, THREADS from the number of rows (one lane per thread for few rows,
// so that every load of a row is in flight at once; 256 threads that play LANES / 256 lanes each for many rows),
// and both give the same bits.  Every pointer is 16-byte aligned, the width a multiple of 4, at most
// MAX_UNROLLED_SPLITS partial sums per sublayer.
template <int LANES, int THREADS>
__device__ __forceinline__ float lanes_total(const float (&mine)[LANES / THREADS], float* warp_partial) {
    constexpr int PLAYED = LANES / THREADS;
#pragma unroll
    for (int k = 0; k < PLAYED; ++k) {
        const float warp_total = warp_sum(mine[k]);
        if ((threadIdx.x & 31) == 0) warp_partial[k * (THREADS / 32) + (threadIdx.x >> 5)] = warp_total;
    }
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < LANES / 32; ++w) total += warp_partial[w];
    __syncthreads();
    return total;
}

__device__ __forceinline__ void add4(float4& a, const float4& b) { a.x += b.x, a.y += b.y, a.z += b.z, a.w += b.w; }

template <typename OutT, int LANES, int THREADS>
__global__ void __launch_bounds__(THREADS) add_layernorm_vec_kernel(LayerNormArgs a) {
    constexpr int PLAYED = LANES / THREADS;
    extern __shared__ float row_cache[];  // [hidden]
    __shared__ float warp_partial[LANES / 32];
    const int out_row = blockIdx.x;
    pdl_trigger();
    const int src = a.rows ? a.rows[out_row] : out_row;
    pdl_wait();
    const size_t offset = static_cast<size_t>(src) * a.hidden;
    float* x_row = a.x + offset;
    const bool write_back = !a.rows && (a.first_splits > 0 || a.second_splits > 0 || a.add_bias != nullptr);
    float sums[PLAYED];
#pragma unroll
    for (int k = 0; k < PLAYED; ++k) sums[k] = 0.0f;
    for (int base = 0; base < a.hidden; base += LANES * 4) {
#pragma unroll
        for (int k = 0; k < PLAYED; ++k) {
            const int i = base + (k * THREADS + threadIdx.x) * 4;
            if (i >= a.hidden) continue;
            float4 v = *reinterpret_cast<const float4*>(x_row + i);
            float4 one[MAX_UNROLLED_SPLITS], two[MAX_UNROLLED_SPLITS];
#pragma unroll
            for (int s = 0; s < MAX_UNROLLED_SPLITS; ++s) {
                if (s < a.first_splits) one[s] = *reinterpret_cast<const float4*>(a.first + s * a.first_stride + offset + i);
                if (s < a.second_splits) two[s] = *reinterpret_cast<const float4*>(a.second + s * a.second_stride + offset + i);
            }
            float4 bias = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (a.add_bias) bias = *reinterpret_cast<const float4*>(a.add_bias + i);
            if (a.first_splits > 0) {
                float4 part = one[0];
#pragma unroll
                for (int s = 1; s < MAX_UNROLLED_SPLITS; ++s)
                    if (s < a.first_splits) add4(part, one[s]);
                if (a.add_bias) add4(part, bias);
                add4(v, part);
            } else if (a.add_bias) {
                add4(v, bias);
            }
            if (a.second_splits > 0) {
                float4 part = two[0];
#pragma unroll
                for (int s = 1; s < MAX_UNROLLED_SPLITS; ++s)
                    if (s < a.second_splits) add4(part, two[s]);
                add4(v, part);
            }
            *reinterpret_cast<float4*>(row_cache + i) = v;
            if (write_back) *reinterpret_cast<float4*>(x_row + i) = v;
            sums[k] += (v.x + v.y) + (v.z + v.w);
        }
    }
    const float mean = lanes_total<LANES, THREADS>(sums, warp_partial) / static_cast<float>(a.hidden);
#pragma unroll
    for (int k = 0; k < PLAYED; ++k) sums[k] = 0.0f;
    for (int base = 0; base < a.hidden; base += LANES * 4) {
#pragma unroll
        for (int k = 0; k < PLAYED; ++k) {
            const int i = base + (k * THREADS + threadIdx.x) * 4;
            if (i >= a.hidden) continue;
            const float4 v = *reinterpret_cast<const float4*>(row_cache + i);
            const float dx = v.x - mean, dy = v.y - mean, dz = v.z - mean, dw = v.w - mean;
            sums[k] = fmaf(dx, dx, sums[k]), sums[k] = fmaf(dy, dy, sums[k]);
            sums[k] = fmaf(dz, dz, sums[k]), sums[k] = fmaf(dw, dw, sums[k]);
        }
    }
    const float inv = rsqrtf(lanes_total<LANES, THREADS>(sums, warp_partial) / static_cast<float>(a.hidden) + a.eps);
    OutT* out_ptr = static_cast<OutT*>(a.out) + static_cast<size_t>(out_row) * a.hidden;
    for (int i = threadIdx.x * 4; i < a.hidden; i += THREADS * 4) {
        const float4 v = *reinterpret_cast<const float4*>(row_cache + i);
        const float4 w = *reinterpret_cast<const float4*>(a.weight + i), b = *reinterpret_cast<const float4*>(a.bias + i);
        store4(out_ptr + i, make_float4(fmaf((v.x - mean) * inv, w.x, b.x), fmaf((v.y - mean) * inv, w.y, b.y),
                                        fmaf((v.z - mean) * inv, w.z, b.z), fmaf((v.w - mean) * inv, w.w, b.w)));
    }
}

template <typename OutT, int LANES, int THREADS>
static int launch_add_layernorm_vec(const LayerNormArgs& a, int count, cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(a.hidden) * sizeof(float);
    auto kernel = add_layernorm_vec_kernel<OutT, LANES, THREADS>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_kernel(kernel, count, THREADS, smem, stream, a);
}

template <typename OutT>
static int launch_add_layernorm_lanes(const LayerNormArgs& a, int count, cudaStream_t stream) {
    const bool many = count >= NORM_MANY_ROWS;
    if (a.hidden > 2048)  // (a block of 1,024 threads has 64 registers a thread, fewer than a lane's loads in flight need)
        return many ? launch_add_layernorm_vec<OutT, 1024, 256>(a, count, stream) : launch_add_layernorm_vec<OutT, 1024, 512>(a, count, stream);
    if (a.hidden > 1024)
        return many ? launch_add_layernorm_vec<OutT, 512, 256>(a, count, stream) : launch_add_layernorm_vec<OutT, 512, 512>(a, count, stream);
    return launch_add_layernorm_vec<OutT, 256, 256>(a, count, stream);
}

ME_EXPORT int me_add_layernorm(float* x, const float* first, int first_splits, long long first_stride,
                               const float* second, int second_splits, long long second_stride, const float* add_bias,
                               const float* weight, const float* bias, float eps, void* out, int out_type,
                               const int* rows, int count, int hidden, cudaStream_t stream) {
    if (count <= 0) return 0;
    const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
    if (smem > 200 * 1024) return ME_ERR_UNSUPPORTED;
    if ((first_splits > 0 && first == nullptr) || (second_splits > 0 && second == nullptr)) return ME_ERR_ARGUMENT;
    LayerNormArgs a{x, first, first_splits, (size_t)first_stride, second, second_splits, (size_t)second_stride,
                    add_bias, weight, bias, eps, out, rows, hidden};
    // Which kernel runs depends on the width, on the alignment of the engine's persistent buffers and on whether
    // the products were split more than eight ways, never on the rows of the step.
    const bool vec = hidden % 4 == 0 && aligned16(x) && aligned16(weight) && aligned16(bias) && aligned16(out) &&
                     aligned16(add_bias) && first_splits <= MAX_UNROLLED_SPLITS && second_splits <= MAX_UNROLLED_SPLITS &&
                     (first_splits == 0 || (aligned16(first) && first_stride % 4 == 0)) &&
                     (second_splits == 0 || (aligned16(second) && second_stride % 4 == 0));
    if (vec)
        return out_type == ME_BF16 ? launch_add_layernorm_lanes<__nv_bfloat16>(a, count, stream)
                                   : launch_add_layernorm_lanes<float>(a, count, stream);
    if (out_type == ME_BF16) {
        auto kernel = add_layernorm_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_kernel(kernel, count, 256, smem, stream, a);
    }
    auto kernel = add_layernorm_kernel<float>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_kernel(kernel, count, 256, smem, stream, a);
}

// --------------------------------------------------------------------------------- SwiGLU

// partial[s][t][0..inter) are gate sums, [inter..2*inter) up sums.  out = g * sigmoid(slope * g) * (u + offset)
// with g = min(gate, limit) and u = clamp(up, -limit, limit) when limit > 0, else g = gate and u = up;
// slope 1, no limit and offset 0 are silu(gate) * up.  With `group_weight [tokens][groups]` the features form
// `groups` equal runs (the units of a routed feed-forward side by side) and feature i of token t is multiplied
// by group_weight[t][i / group_size].  `activation` 1 replaces g * sigmoid(slope * g) by the tanh form of GELU,
// 0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3))).
enum : int { GATE_SIGMOID = 0, GATE_GELU_TANH = 1 };

__device__ __forceinline__ float gate_activation(float g, float slope, int activation) {
    if (activation == GATE_GELU_TANH) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return g / (1.0f + expf(-slope * g));
}

template <typename OutT>
__global__ void swiglu_kernel(const float* __restrict__ partial, int splits, size_t split_stride,
                              OutT* __restrict__ out, int tokens, int inter, float slope, float limit, float offset,
                              const float* __restrict__ group_weight, int group_size, int groups, int activation) {
    const size_t total = static_cast<size_t>(tokens) * inter;
    pdl_trigger();
    pdl_wait();
    for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t t = idx / inter;
        const size_t i = idx - t * inter;
        const float* base = partial + t * 2 * inter;
        float gate = 0.0f, up = 0.0f;
        for (int s = 0; s < splits; ++s) {
            gate += base[s * split_stride + i];
            up += base[s * split_stride + inter + i];
        }
        if (limit > 0.0f) {
            gate = fminf(gate, limit);
            up = fminf(fmaxf(up, -limit), limit);
        }
        const float activated = gate_activation(gate, slope, activation);
        float value = activated * (up + offset);
        // routed units: feature i belongs to unit i / group_size, whose weight for this token may be zero
        if (group_weight != nullptr) value *= group_weight[t * groups + i / group_size];
        out[idx] = from_float<OutT>(value);
    }
}

// The same with four consecutive features per thread (16-byte loads): widths that are multiples of 4, groups too.
template <typename OutT>
__global__ void swiglu_vec_kernel(const float* __restrict__ partial, int splits, size_t split_stride,
                                  OutT* __restrict__ out, int tokens, int inter, float slope, float limit, float offset,
                                  const float* __restrict__ group_weight, int group_size, int groups, int activation) {
    const size_t quads = static_cast<size_t>(inter / 4);
    const size_t total = static_cast<size_t>(tokens) * quads;
    pdl_trigger();
    pdl_wait();
    for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t t = idx / quads;
        const size_t i = (idx - t * quads) * 4;
        const float* base = partial + t * 2 * inter + i;
        float4 gate = make_float4(0.0f, 0.0f, 0.0f, 0.0f), up = gate;
        for (int s = 0; s < splits; ++s) {
            const float4 g = *reinterpret_cast<const float4*>(base + s * split_stride);
            const float4 u = *reinterpret_cast<const float4*>(base + s * split_stride + inter);
            gate.x += g.x, gate.y += g.y, gate.z += g.z, gate.w += g.w;
            up.x += u.x, up.y += u.y, up.z += u.z, up.w += u.w;
        }
        const float weight = group_weight != nullptr ? group_weight[t * groups + i / group_size] : 1.0f;
        float g4[4] = {gate.x, gate.y, gate.z, gate.w}, u4[4] = {up.x, up.y, up.z, up.w}, y[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float g = g4[j], u = u4[j];
            if (limit > 0.0f) {
                g = fminf(g, limit);
                u = fminf(fmaxf(u, -limit), limit);
            }
            const float activated = gate_activation(g, slope, activation);
            y[j] = activated * (u + offset);
            if (group_weight != nullptr) y[j] *= weight;
        }
        store4(out + t * inter + i, make_float4(y[0], y[1], y[2], y[3]));
    }
}

ME_EXPORT int me_swiglu(const float* partial, int splits, long long split_stride, void* out, int out_type,
                        int tokens, int inter, float slope, float limit, float offset, const float* group_weight,
                        int group_size, int activation, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (activation != GATE_SIGMOID && activation != GATE_GELU_TANH) return ME_ERR_ARGUMENT;
    if (group_weight != nullptr && (group_size < 1 || inter % group_size)) return ME_ERR_ARGUMENT;
    const int groups = group_weight != nullptr ? inter / group_size : 0;
    const size_t total = static_cast<size_t>(tokens) * inter;
    const int threads = 256;
    // The choice depends on the sizes and the engine's buffers only; both forms give an element the same bits.
    const bool vec = inter % 4 == 0 && split_stride % 4 == 0 && reinterpret_cast<uintptr_t>(partial) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(out) % 16 == 0 && (group_weight == nullptr || group_size % 4 == 0);
    if (vec) {
        const int blocks = static_cast<int>(std::min<size_t>((total / 4 + threads - 1) / threads, 148 * 64));
        if (out_type == ME_BF16)
            return launch_kernel(swiglu_vec_kernel<__nv_bfloat16>, blocks, threads, 0, stream, partial, splits, (size_t)split_stride,
                                 static_cast<__nv_bfloat16*>(out), tokens, inter, slope, limit, offset, group_weight, group_size, groups, activation);
        return launch_kernel(swiglu_vec_kernel<float>, blocks, threads, 0, stream, partial, splits, (size_t)split_stride,
                             static_cast<float*>(out), tokens, inter, slope, limit, offset, group_weight, group_size, groups, activation);
    }
    const int blocks = static_cast<int>(std::min<size_t>((total + threads - 1) / threads, 148 * 16));
    if (out_type == ME_BF16)
        return launch_kernel(swiglu_kernel<__nv_bfloat16>, blocks, threads, 0, stream, partial, splits,
                             (size_t)split_stride, static_cast<__nv_bfloat16*>(out), tokens, inter, slope, limit, offset,
                             group_weight, group_size, groups, activation);
    return launch_kernel(swiglu_kernel<float>, blocks, threads, 0, stream, partial, splits, (size_t)split_stride,
                         static_cast<float*>(out), tokens, inter, slope, limit, offset, group_weight, group_size, groups, activation);
}

// ------------------------------------------------- per-head norm + rotary + cache write

// One warp per (token, head) over the columns of qkv = [q heads | k heads | v heads].
//   q heads: optional RMSNorm over head_dim, optional rotation, written to q_out[t][h][:].
//   k heads: the same, written to the token's slot of k_pages (or to k_dense[t][h][:]).
//   v heads: copied to the slot of v_pages (or v_dense).
// Pages are [page][kv_head][slot in page][head_dim]; slot_mapping[t] = page * page_size + slot,
// negative for a token whose keys are not to be stored.
struct QkvArgs {
    const float* qkv;     // [splits][tokens][(heads + 2 kv_heads) * head_dim]
    int splits;
    size_t split_stride;
    const float* q_weight;  // [head_dim] or null: no norm
    const float* k_weight;
    float eps;
    const float2* cos_sin;  // [tokens][rotary_dim / 2] (cos, sin) of each token's angles, or null: no rotation
    const int* positions;
    const int* slot_mapping;  // null: dense outputs
    void* q_out;
    void* k_pages;
    void* v_pages;
    void* k_dense;
    void* v_dense;
    int tokens, heads, kv_heads, head_dim, page_size;
    int rotary_dim;  // the first rotary_dim elements of a head are rotated (in halves of rotary_dim / 2), the rest pass through
    const float* bias;  // [(heads + 2 kv_heads) * head_dim] added to the projections' sums, or null
    int value_dim;      // width of a value head (head_dim in most models): the v columns are kv_heads * value_dim
};

constexpr int QKV_WARPS = 4;
constexpr int MAX_HEAD_DIM = 512;

template <typename OutT>
__global__ void __launch_bounds__(QKV_WARPS * 32) qk_norm_rope_store_kernel(QkvArgs a) {
    extern __shared__ float staged[];  // [QKV_WARPS][head_dim]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = a.heads + 2 * a.kv_heads;
    const long long item = static_cast<long long>(blockIdx.x) * QKV_WARPS + warp;
    if (item >= static_cast<long long>(a.tokens) * heads_total) return;
    const int token = static_cast<int>(item / heads_total);
    const int column_head = static_cast<int>(item % heads_total);
    const int half = a.rotary_dim / 2;
    const bool is_q = column_head < a.heads;
    const bool is_k = !is_q && column_head < a.heads + a.kv_heads;
    // Query and key heads are head_dim wide, value heads value_dim.
    const int d = (is_q || is_k) ? a.head_dim : a.value_dim;
    float* vec = staged + warp * max(a.head_dim, a.value_dim);
    pdl_trigger();
    pdl_wait();

    const size_t qk_heads = static_cast<size_t>(a.heads + a.kv_heads);
    const size_t row_width = qk_heads * a.head_dim + static_cast<size_t>(a.kv_heads) * a.value_dim;
    const size_t column = (is_q || is_k) ? static_cast<size_t>(column_head) * a.head_dim
                                         : qk_heads * a.head_dim + (column_head - qk_heads) * a.value_dim;
    const float* src = a.qkv + static_cast<size_t>(token) * row_width + column;
    float sum_sq = 0.0f;
    for (int i = lane; i < d; i += 32) {
        float v = 0.0f;
        for (int s = 0; s < a.splits; ++s) v += src[s * a.split_stride + i];
        if (a.bias) v += a.bias[column + i];
        vec[i] = v;
        sum_sq = fmaf(v, v, sum_sq);
    }
    const float* weight = is_q ? a.q_weight : (is_k ? a.k_weight : nullptr);
    float inv = 1.0f;
    if (weight) {
        sum_sq = warp_sum(sum_sq);
        inv = rsqrtf(sum_sq / static_cast<float>(d) + a.eps);
    }
    __syncwarp();

    OutT* dst;
    if (is_q) {
        dst = static_cast<OutT*>(a.q_out) + (static_cast<size_t>(token) * a.heads + column_head) * d;
    } else {
        const int kv_head = is_k ? column_head - a.heads : column_head - a.heads - a.kv_heads;
        if (a.slot_mapping) {
            const int slot = a.slot_mapping[token];
            if (slot < 0) return;
            const size_t page = slot / a.page_size, offset = slot % a.page_size;
            OutT* pages = static_cast<OutT*>(is_k ? a.k_pages : a.v_pages);
            dst = pages + ((page * a.kv_heads + kv_head) * a.page_size + offset) * d;
        } else {
            OutT* dense = static_cast<OutT*>(is_k ? a.k_dense : a.v_dense);
            dst = dense + (static_cast<size_t>(token) * a.kv_heads + kv_head) * d;
        }
    }
    const bool rotate = (is_q || is_k) && a.cos_sin != nullptr;
    const float2* angles = a.cos_sin + static_cast<size_t>(token) * half;
    for (int i = lane; i < d; i += 32) {
        float value = weight ? weight[i] * (vec[i] * inv) : vec[i];
        if (rotate && i < a.rotary_dim) {
            // rotate-half: out[i] = x[i] cos - x[i + half] sin (i < half); x[i] cos + x[i - half] sin.
            const int j = i < half ? i + half : i - half;
            const float other = weight ? weight[j] * (vec[j] * inv) : vec[j];
            const float2 angle = angles[i < half ? i : i - half];
            const float cosine = angle.x, sine = angle.y;
            value = i < half ? value * cosine - other * sine : value * cosine + other * sine;
        }
        dst[i] = from_float<OutT>(value);
    }
}

// The same for head_dim == 128: each lane owns four consecutive elements, all partial sums are
// loaded before they are added, and the rotation partner (64 elements away) is 16 lanes away.
// A warp takes HEADS consecutive heads of one token and requests all of them before it uses any:
// with one partial sum (prompts) four heads per warp keep enough loads in flight to fill HBM.
template <typename OutT, int HEADS, int MAX_SPLITS>
__global__ void __launch_bounds__(QKV_WARPS * 32) qk_norm_rope_store_128_kernel(QkvArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = a.heads + 2 * a.kv_heads;
    const int groups = heads_total / HEADS;  // the launcher makes sure this divides
    const long long item = static_cast<long long>(blockIdx.x) * QKV_WARPS + warp;
    if (item >= static_cast<long long>(a.tokens) * groups) return;
    const int token = static_cast<int>(item / groups);
    const int first_head = static_cast<int>(item % groups) * HEADS;
    constexpr int D = 128;
    pdl_trigger();
    // Weights and the step's slot list do not come from the previous kernel: fetch them ahead of the wait.
    const float4 one = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
    const float4 q_w = a.q_weight ? *reinterpret_cast<const float4*>(a.q_weight + lane * 4) : one;
    const float4 k_w = a.k_weight ? *reinterpret_cast<const float4*>(a.k_weight + lane * 4) : one;
    const int slot = a.slot_mapping ? a.slot_mapping[token] : 0;
    pdl_wait();
    const float* src = a.qkv + static_cast<size_t>(token) * heads_total * D + static_cast<size_t>(first_head) * D + lane * 4;
    float4 part[HEADS][MAX_SPLITS];
#pragma unroll
    for (int u = 0; u < HEADS; ++u)
#pragma unroll
        for (int s = 0; s < MAX_SPLITS; ++s)
            if (s < a.splits) part[u][s] = *reinterpret_cast<const float4*>(src + u * D + s * a.split_stride);
    float4 first = make_float4(1.0f, 0.0f, 1.0f, 0.0f), second = first;
    if (a.cos_sin != nullptr) {
        const float4* angles = reinterpret_cast<const float4*>(a.cos_sin + static_cast<size_t>(token) * (D / 2) + (lane & 15) * 4);
        first = angles[0];   // (cos, sin) of four consecutive frequencies
        second = angles[1];
    }
#pragma unroll
    for (int u = 0; u < HEADS; ++u) {
        const int column_head = first_head + u;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int s = 0; s < MAX_SPLITS; ++s)
            if (s < a.splits) { v.x += part[u][s].x; v.y += part[u][s].y; v.z += part[u][s].z; v.w += part[u][s].w; }
        if (a.bias) {
            const float4 b = *reinterpret_cast<const float4*>(a.bias + static_cast<size_t>(column_head) * D + lane * 4);
            v.x += b.x, v.y += b.y, v.z += b.z, v.w += b.w;
        }
        const bool is_q = column_head < a.heads;
        const bool is_k = !is_q && column_head < a.heads + a.kv_heads;
        const float* weight = is_q ? a.q_weight : (is_k ? a.k_weight : nullptr);
        if (weight) {
            float sum_sq = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
            sum_sq = warp_sum(sum_sq);
            const float inv = rsqrtf(sum_sq / static_cast<float>(D) + a.eps);
            const float4 w = is_q ? q_w : k_w;
            v = make_float4(w.x * (v.x * inv), w.y * (v.y * inv), w.z * (v.z * inv), w.w * (v.w * inv));
        }
        if ((is_q || is_k) && a.cos_sin != nullptr) {
            const float4 other = make_float4(__shfl_xor_sync(0xffffffffu, v.x, 16), __shfl_xor_sync(0xffffffffu, v.y, 16),
                                             __shfl_xor_sync(0xffffffffu, v.z, 16), __shfl_xor_sync(0xffffffffu, v.w, 16));
            const float sign = lane < 16 ? -1.0f : 1.0f;  // first half: x cos - partner sin; second: x cos + partner sin
            v.x = v.x * first.x + sign * other.x * first.y;
            v.y = v.y * first.z + sign * other.y * first.w;
            v.z = v.z * second.x + sign * other.z * second.y;
            v.w = v.w * second.z + sign * other.w * second.w;
        }
        OutT* dst;
        if (is_q) {
            dst = static_cast<OutT*>(a.q_out) + (static_cast<size_t>(token) * a.heads + column_head) * D;
        } else {
            const int kv_head = is_k ? column_head - a.heads : column_head - a.heads - a.kv_heads;
            if (a.slot_mapping) {
                if (slot < 0) continue;
                const size_t page = slot / a.page_size, offset = slot % a.page_size;
                OutT* pages = static_cast<OutT*>(is_k ? a.k_pages : a.v_pages);
                dst = pages + ((page * a.kv_heads + kv_head) * a.page_size + offset) * D;
            } else {
                OutT* dense = static_cast<OutT*>(is_k ? a.k_dense : a.v_dense);
                dst = dense + (static_cast<size_t>(token) * a.kv_heads + kv_head) * D;
            }
        }
        store4(dst + lane * 4, v);
    }
}

// (cos, sin) of position * inv_freq for every token of the step, once per step for all layers
// (src/mini_engine/model.py:79-83,183 of YuvGev00/mini-engine builds its tables once per step too).
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                  float2* __restrict__ out, int tokens, int half) {
    pdl_trigger();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= tokens * half) return;
    const int token = idx / half, i = idx % half;
    float sine, cosine;
    sincosf(static_cast<float>(positions[token]) * inv_freq[i], &sine, &cosine);
    out[idx] = make_float2(cosine, sine);
}

ME_EXPORT int me_rope_table(const float* inv_freq, const int* positions, float* out, int tokens, int half,
                            cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const int total = tokens * half;
    return launch_kernel(rope_table_kernel, (total + 255) / 256, 256, 0, stream, inv_freq, positions,
                         reinterpret_cast<float2*>(out), tokens, half);
}

ME_EXPORT int me_qk_norm_rope_store(const float* qkv, int splits, long long split_stride, const float* q_weight,
                                    const float* k_weight, float eps, const float* cos_sin,
                                    const int* positions, const int* slot_mapping, void* q_out, void* k_pages,
                                    void* v_pages, void* k_dense, void* v_dense, int out_type, int tokens,
                                    int heads, int kv_heads, int head_dim, int page_size, int rotary_dim,
                                    const float* bias, int value_dim, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (head_dim > MAX_HEAD_DIM || (head_dim % 2 && cos_sin != nullptr)) return ME_ERR_UNSUPPORTED;
    if (value_dim < 1 || value_dim > MAX_HEAD_DIM) return ME_ERR_UNSUPPORTED;
    if (rotary_dim < 0 || rotary_dim > head_dim || rotary_dim % 2) return ME_ERR_ARGUMENT;
    QkvArgs a{qkv, splits, (size_t)split_stride, q_weight, k_weight, eps, reinterpret_cast<const float2*>(cos_sin), positions, slot_mapping,
              q_out, k_pages, v_pages, k_dense, v_dense, tokens, heads, kv_heads, head_dim, page_size, rotary_dim, bias, value_dim};
    const long long items = static_cast<long long>(tokens) * (heads + 2 * kv_heads);
    const int blocks = static_cast<int>((items + QKV_WARPS - 1) / QKV_WARPS);
    const size_t smem = static_cast<size_t>(QKV_WARPS) * std::max(head_dim, value_dim) * sizeof(float);
    // The choice depends on the model's sizes and the engine's buffers only, never on the batch.
    const bool vec = head_dim == 128 && value_dim == 128 && rotary_dim == head_dim && splits <= MAX_UNROLLED_SPLITS && split_stride % 4 == 0 && aligned16(qkv) &&
                     aligned16(q_out) && aligned16(k_pages) && aligned16(v_pages) && aligned16(k_dense) &&
                     aligned16(v_dense) && aligned16(q_weight) && aligned16(k_weight) && aligned16(cos_sin) && aligned16(bias);
    if (vec) {
        // The number of heads per warp depends on the number of partial sums and on the model's
        // head counts only, never on the batch.
        const bool four = splits == 1 && (heads + 2 * kv_heads) % 4 == 0;
        const long long warps = static_cast<long long>(tokens) * ((heads + 2 * kv_heads) / (four ? 4 : 1));
        const int vec_blocks = static_cast<int>((warps + QKV_WARPS - 1) / QKV_WARPS);
        if (out_type == ME_BF16)
            return four ? launch_kernel(qk_norm_rope_store_128_kernel<__nv_bfloat16, 4, 1>, vec_blocks, QKV_WARPS * 32, 0, stream, a)
                        : launch_kernel(qk_norm_rope_store_128_kernel<__nv_bfloat16, 1, MAX_UNROLLED_SPLITS>, vec_blocks, QKV_WARPS * 32, 0, stream, a);
        return four ? launch_kernel(qk_norm_rope_store_128_kernel<float, 4, 1>, vec_blocks, QKV_WARPS * 32, 0, stream, a)
                    : launch_kernel(qk_norm_rope_store_128_kernel<float, 1, MAX_UNROLLED_SPLITS>, vec_blocks, QKV_WARPS * 32, 0, stream, a);
    }
    if (out_type == ME_BF16)
        return launch_kernel(qk_norm_rope_store_kernel<__nv_bfloat16>, blocks, QKV_WARPS * 32, smem, stream, a);
    return launch_kernel(qk_norm_rope_store_kernel<float>, blocks, QKV_WARPS * 32, smem, stream, a);
}

// Dense [tokens][kv_heads][head_dim] keys and values into their slots of the pages.
template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ k_dense, const T* __restrict__ v_dense,
                                const int* __restrict__ slot_mapping, T* __restrict__ k_pages,
                                T* __restrict__ v_pages, int kv_heads, int head_dim, int page_size) {
    const int token = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    const int slot = slot_mapping[token];
    if (slot < 0) return;
    const size_t page = slot / page_size, offset = slot % page_size;
    const int width = kv_heads * head_dim;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const int head = i / head_dim, e = i % head_dim;
        const size_t dst = ((page * kv_heads + head) * page_size + offset) * head_dim + e;
        k_pages[dst] = k_dense[static_cast<size_t>(token) * width + i];
        v_pages[dst] = v_dense[static_cast<size_t>(token) * width + i];
    }
}

ME_EXPORT int me_kv_store(const void* k_dense, const void* v_dense, const int* slot_mapping, void* k_pages,
                          void* v_pages, int type, int tokens, int kv_heads, int head_dim, int page_size,
                          cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (type == ME_BF16)
        return launch_kernel(kv_store_kernel<__nv_bfloat16>, tokens, 128, 0, stream,
                             static_cast<const __nv_bfloat16*>(k_dense), static_cast<const __nv_bfloat16*>(v_dense),
                             slot_mapping, static_cast<__nv_bfloat16*>(k_pages), static_cast<__nv_bfloat16*>(v_pages),
                             kv_heads, head_dim, page_size);
    return launch_kernel(kv_store_kernel<float>, tokens, 128, 0, stream, static_cast<const float*>(k_dense),
                         static_cast<const float*>(v_dense), slot_mapping, static_cast<float*>(k_pages),
                         static_cast<float*>(v_pages), kv_heads, head_dim, page_size);
}

// ------------------------------------------------------- weighted sum of parallel branches

// out[t][c] = sum_b factor[b] * (sum_s partial_b[s][t][c]): the outputs of mixers that read the same
// input side by side, each still in the partial sums of its last product, joined into one float32 array.
constexpr int MAX_BRANCHES = 4;
struct BranchArgs {
    const float* partial[MAX_BRANCHES];
    int splits[MAX_BRANCHES];
    size_t split_stride[MAX_BRANCHES];
    float factor[MAX_BRANCHES];
    int branches;
};

__global__ void branch_sum_kernel(BranchArgs a, float* __restrict__ out, size_t total) {
    pdl_trigger();
    pdl_wait();
    for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float sum = 0.0f;
        for (int b = 0; b < a.branches; ++b) {
            float whole = 0.0f;
            for (int s = 0; s < a.splits[b]; ++s) whole += a.partial[b][s * a.split_stride[b] + idx];
            sum = fmaf(a.factor[b], whole, sum);
        }
        out[idx] = sum;
    }
}

ME_EXPORT int me_branch_sum(const float* const* partials, const int* splits, const long long* strides,
                            const float* factors, int branches, float* out, int tokens, int width,
                            cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (branches < 1 || branches > MAX_BRANCHES) return ME_ERR_UNSUPPORTED;
    BranchArgs a{};
    a.branches = branches;
    for (int b = 0; b < branches; ++b) {
        a.partial[b] = partials[b];
        a.splits[b] = splits[b];
        a.split_stride[b] = static_cast<size_t>(strides[b]);
        a.factor[b] = factors[b];
    }
    const size_t total = static_cast<size_t>(tokens) * width;
    const int threads = 256;
    const int blocks = static_cast<int>(std::min<size_t>((total + threads - 1) / threads, 148 * 16));
    return launch_kernel(branch_sum_kernel, blocks, threads, 0, stream, a, out, total);
}

// --------------------------------------------------- embedding with a second, pair-hashed table

// out[t] = table[id_t] * multiplier + pair_table[row_t], float32, one block per token.  row_t is
// (previous id * mul_prev + id_t * mul_cur) mod buckets, and `buckets` (the table's last row) for the
// first token of a sequence.  The previous id of an entry's first token is the request's state
// (last_token[slot]; nothing when the entry starts its sequence); the block of an entry's first token
// also leaves the entry's last id there for the next step.  `rounded` (optional) receives the same row
// in the compute dtype for a first layer that reads the stream itself.
struct PairEmbeddingArgs {
    const void* table;
    const void* pair_table;
    const int* ids;
    const int* entry_of_token;
    const int* cu_tokens;
    const int* state_slots;
    const int* fresh;
    int* last_token;  // [slots + 1]
    float* out;
    void* rounded;
    int hidden, vocab, buckets;
    long long mul_prev, mul_cur;
    float multiplier;
};

template <typename T, typename RoundT>
__global__ void pair_embedding_kernel(PairEmbeddingArgs a) {
    const int token = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    const int id = a.ids[token];
    const int entry = a.entry_of_token[token];
    const int first = a.cu_tokens[entry];
    int previous = -1;
    if (token != first) previous = a.ids[token - 1];
    else if (!a.fresh[entry]) previous = a.last_token[a.state_slots[entry]];
    __syncthreads();  // every thread has read the state before one of them replaces it
    if (token == first && threadIdx.x == 0) a.last_token[a.state_slots[entry]] = a.ids[a.cu_tokens[entry + 1] - 1];
    float* row_out = a.out + static_cast<size_t>(token) * a.hidden;
    RoundT* row_rounded = a.rounded ? static_cast<RoundT*>(a.rounded) + static_cast<size_t>(token) * a.hidden : nullptr;
    if (id < 0 || id >= a.vocab) {  // the host validates ids; never read outside the table
        for (int i = threadIdx.x; i < a.hidden; i += blockDim.x) {
            row_out[i] = 0.0f;
            if (row_rounded) row_rounded[i] = from_float<RoundT>(0.0f);
        }
        return;
    }
    long long pair = a.buckets;
    if (previous >= 0) pair = (previous * a.mul_prev + id * a.mul_cur) % a.buckets;
    const T* row = static_cast<const T*>(a.table) + static_cast<size_t>(id) * a.hidden;
    const T* pair_row = static_cast<const T*>(a.pair_table) + static_cast<size_t>(pair) * a.hidden;
    for (int i = threadIdx.x; i < a.hidden; i += blockDim.x) {
        const float value = __fadd_rn(__fmul_rn(to_float(row[i]), a.multiplier), to_float(pair_row[i]));
        row_out[i] = value;
        if (row_rounded) row_rounded[i] = from_float<RoundT>(value);
    }
}

ME_EXPORT int me_pair_embedding(const void* table, const void* pair_table, int table_type, const int* ids,
                                const int* entry_of_token, const int* cu_tokens, const int* state_slots,
                                const int* fresh, int* last_token, float* out, void* rounded, int rounded_type,
                                int tokens, int hidden, int vocab, int buckets, long long mul_prev, long long mul_cur,
                                float multiplier, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (buckets < 1 || mul_prev < 0 || mul_cur < 0) return ME_ERR_ARGUMENT;
    PairEmbeddingArgs a{table, pair_table, ids, entry_of_token, cu_tokens, state_slots, fresh, last_token, out, rounded,
                        hidden, vocab, buckets, mul_prev, mul_cur, multiplier};
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_type == ME_BF16) {
        if (rounded_type == ME_BF16) return launch_kernel(pair_embedding_kernel<__nv_bfloat16, __nv_bfloat16>, tokens, threads, 0, stream, a);
        return launch_kernel(pair_embedding_kernel<__nv_bfloat16, float>, tokens, threads, 0, stream, a);
    }
    if (rounded_type == ME_BF16) return launch_kernel(pair_embedding_kernel<float, __nv_bfloat16>, tokens, threads, 0, stream, a);
    return launch_kernel(pair_embedding_kernel<float, float>, tokens, threads, 0, stream, a);
}

// ------------------------------------------------------------------------ float32 rows, rounded

template <typename OutT>
__global__ void round_rows_kernel(const float* __restrict__ x, OutT* __restrict__ out, size_t total) {
    pdl_trigger();
    pdl_wait();
    for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x)
        out[idx] = from_float<OutT>(x[idx]);
}

// out = x in the compute dtype: the input of a sublayer that reads the residual stream itself.
ME_EXPORT int me_round_rows(const float* x, void* out, int out_type, int rows, int width, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const size_t total = static_cast<size_t>(rows) * width;
    const int blocks = static_cast<int>(std::min<size_t>((total + 255) / 256, 148 * 16));
    if (out_type == ME_BF16)
        return launch_kernel(round_rows_kernel<__nv_bfloat16>, blocks, 256, 0, stream, x, static_cast<__nv_bfloat16*>(out), total);
    return launch_kernel(round_rows_kernel<float>, blocks, 256, 0, stream, x, static_cast<float*>(out), total);
}

// ------------------------------------- norm over a whole projection + rotary + cache write + gates

// One block per token over the columns of qkv = [q heads | k heads | v heads | gates].  Unlike the per-head
// kernel above, q is normalised over all of its heads * head_dim columns at once with a weight of that size,
// and k over its kv_heads * head_dim columns; then each head's first rotary_dim elements are rotated, q goes to
// q_out and k, v to the token's cache slot (or to dense buffers).  `gates` trailing columns (one per query
// head in the models that have them) leave the kernel as sigmoid(sum) in gate_out[t][gates], float32.
// kv_heads == 0: a layer that reads another layer's keys and values has no k and v columns.  `bias` (one value
// per column of the row, gates included) is added to the sums first.
struct WideQkvArgs {
    const float* qkv;  // [splits][tokens][row_width]
    int splits;
    size_t split_stride;
    int row_width;
    const float* q_weight;  // [heads * head_dim] or null
    const float* k_weight;  // [kv_heads * head_dim] or null
    float eps;
    const float2* cos_sin;  // [tokens][rotary_dim / 2] or null
    const int* slot_mapping;
    void* q_out;
    void* k_pages;
    void* v_pages;
    void* k_dense;
    void* v_dense;
    float* gate_out;
    int tokens, heads, kv_heads, head_dim, value_dim, page_size, rotary_dim, gates;
    const float* bias;  // [row_width] added to the sums before anything else, or null
};

template <typename OutT>
__global__ void __launch_bounds__(256) qk_wide_norm_rope_store_kernel(WideQkvArgs a) {
    extern __shared__ float row[];  // [row_width]
    __shared__ float warp_partial[2][8];
    const int token = blockIdx.x;
    const int q_width = a.heads * a.head_dim, k_width = a.kv_heads * a.head_dim, v_width = a.kv_heads * a.value_dim;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_trigger();
    pdl_wait();
    const float* src = a.qkv + static_cast<size_t>(token) * a.row_width;
    // Column i's square goes to the partial sum of thread i % 256, in ascending order: a token's
    // statistics are the same bits in every step.
    float q_sq = 0.0f, k_sq = 0.0f;
    for (int i = threadIdx.x; i < a.row_width; i += 256) {
        float v = 0.0f;
        for (int s = 0; s < a.splits; ++s) v += src[s * a.split_stride + i];
        if (a.bias) v += a.bias[i];
        row[i] = v;
        if (i < q_width) q_sq = fmaf(v, v, q_sq);
        else if (i < q_width + k_width) k_sq = fmaf(v, v, k_sq);
    }
    q_sq = warp_sum(q_sq), k_sq = warp_sum(k_sq);
    if (lane == 0) warp_partial[0][warp] = q_sq, warp_partial[1][warp] = k_sq;
    __syncthreads();
    float q_total = 0.0f, k_total = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) q_total += warp_partial[0][w], k_total += warp_partial[1][w];
    const float q_inv = a.q_weight ? rsqrtf(q_total / static_cast<float>(q_width) + a.eps) : 1.0f;
    const float k_inv = (a.k_weight && k_width) ? rsqrtf(k_total / static_cast<float>(k_width) + a.eps) : 1.0f;
    const int half = a.rotary_dim / 2;
    const float2* angles = a.cos_sin ? a.cos_sin + static_cast<size_t>(token) * half : nullptr;
    const int slot = (a.slot_mapping && a.kv_heads) ? a.slot_mapping[token] : -1;
    for (int i = threadIdx.x; i < a.row_width; i += 256) {
        if (i < q_width + k_width) {
            const bool is_q = i < q_width;
            const int column = is_q ? i : i - q_width;
            const int head = column / a.head_dim, e = column % a.head_dim;
            const float* weight = is_q ? a.q_weight : a.k_weight;
            const float inv = is_q ? q_inv : k_inv;
            float value = weight ? weight[column] * (row[i] * inv) : row[i];
            if (angles && e < a.rotary_dim) {
                const int partner = e < half ? i + half : i - half;
                const int partner_column = e < half ? column + half : column - half;
                const float other = weight ? weight[partner_column] * (row[partner] * inv) : row[partner];
                const float2 angle = angles[e < half ? e : e - half];
                value = e < half ? value * angle.x - other * angle.y : value * angle.x + other * angle.y;
            }
            if (is_q) {
                static_cast<OutT*>(a.q_out)[static_cast<size_t>(token) * q_width + column] = from_float<OutT>(value);
            } else if (a.slot_mapping) {
                if (slot >= 0) {
                    const size_t page = slot / a.page_size, offset = slot % a.page_size;
                    static_cast<OutT*>(a.k_pages)[((page * a.kv_heads + head) * a.page_size + offset) * a.head_dim + e] = from_float<OutT>(value);
                }
            } else {
                static_cast<OutT*>(a.k_dense)[static_cast<size_t>(token) * k_width + column] = from_float<OutT>(value);
            }
        } else if (i < q_width + k_width + v_width) {
            const int column = i - q_width - k_width;
            const int head = column / a.value_dim, e = column % a.value_dim;
            if (a.slot_mapping) {
                if (slot >= 0) {
                    const size_t page = slot / a.page_size, offset = slot % a.page_size;
                    static_cast<OutT*>(a.v_pages)[((page * a.kv_heads + head) * a.page_size + offset) * a.value_dim + e] = from_float<OutT>(row[i]);
                }
            } else {
                static_cast<OutT*>(a.v_dense)[static_cast<size_t>(token) * v_width + column] = from_float<OutT>(row[i]);
            }
        } else {
            const int g = i - q_width - k_width - v_width;
            if (g < a.gates) a.gate_out[static_cast<size_t>(token) * a.gates + g] = 1.0f / (1.0f + expf(-row[i]));
        }
    }
}

// The same row without a norm and without a rotation: every column stands alone, so a thread takes four consecutive
// columns of one token (grid: runs of 1,024 columns x tokens), adds their partial sums in ascending order and the
// bias, and stores them where the kernel above would (the same bits).  Every segment of the row starts and ends at a
// multiple of four columns, as does every head; all pointers are 16-byte aligned; at most MAX_UNROLLED_SPLITS sums.
template <typename OutT>
__global__ void __launch_bounds__(256) qkv_bias_store_kernel(WideQkvArgs a) {
    const int token = blockIdx.y;
    const int i = (blockIdx.x * 256 + threadIdx.x) * 4;
    pdl_trigger();
    pdl_wait();
    if (i >= a.row_width) return;
    const float* src = a.qkv + static_cast<size_t>(token) * a.row_width + i;
    float4 part[MAX_UNROLLED_SPLITS];
#pragma unroll
    for (int s = 0; s < MAX_UNROLLED_SPLITS; ++s)
        if (s < a.splits) part[s] = *reinterpret_cast<const float4*>(src + s * a.split_stride);
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int s = 0; s < MAX_UNROLLED_SPLITS; ++s)
        if (s < a.splits) add4(v, part[s]);
    if (a.bias) add4(v, *reinterpret_cast<const float4*>(a.bias + i));
    const int q_width = a.heads * a.head_dim, k_width = a.kv_heads * a.head_dim, v_width = a.kv_heads * a.value_dim;
    if (i < q_width) {
        store4(static_cast<OutT*>(a.q_out) + static_cast<size_t>(token) * q_width + i, v);
    } else if (i < q_width + k_width + v_width) {
        const bool is_k = i < q_width + k_width;
        const int column = is_k ? i - q_width : i - q_width - k_width;
        const int dim = is_k ? a.head_dim : a.value_dim;
        const int head = column / dim, e = column - head * dim;
        if (a.slot_mapping) {
            const int slot = a.slot_mapping[token];
            if (slot < 0) return;
            const size_t page = slot / a.page_size, offset = slot % a.page_size;
            OutT* pages = static_cast<OutT*>(is_k ? a.k_pages : a.v_pages);
            store4(pages + ((page * a.kv_heads + head) * a.page_size + offset) * dim + e, v);
        } else {
            OutT* dense = static_cast<OutT*>(is_k ? a.k_dense : a.v_dense);
            store4(dense + static_cast<size_t>(token) * (is_k ? k_width : v_width) + column, v);
        }
    } else {
        const int g = i - q_width - k_width - v_width;
        if (g < a.gates)
            store4(a.gate_out + static_cast<size_t>(token) * a.gates + g,
                   make_float4(1.0f / (1.0f + expf(-v.x)), 1.0f / (1.0f + expf(-v.y)), 1.0f / (1.0f + expf(-v.z)), 1.0f / (1.0f + expf(-v.w))));
    }
}

ME_EXPORT int me_qk_wide_norm_rope_store(const float* qkv, int splits, long long split_stride, int row_width,
                                         const float* q_weight, const float* k_weight, float eps, const float* cos_sin,
                                         const int* slot_mapping, void* q_out, void* k_pages, void* v_pages,
                                         void* k_dense, void* v_dense, float* gate_out, int out_type, int tokens,
                                         int heads, int kv_heads, int head_dim, int value_dim, int page_size,
                                         int rotary_dim, int gates, const float* bias, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > head_dim || rotary_dim % 2) return ME_ERR_ARGUMENT;
    if (row_width < (heads + kv_heads) * head_dim + kv_heads * value_dim + gates) return ME_ERR_ARGUMENT;
    if (gates > 0 && gate_out == nullptr) return ME_ERR_ARGUMENT;
    const size_t smem = static_cast<size_t>(row_width) * sizeof(float);
    if (smem > 200 * 1024) return ME_ERR_UNSUPPORTED;
    WideQkvArgs a{qkv, splits, (size_t)split_stride, row_width, q_weight, k_weight, eps, reinterpret_cast<const float2*>(cos_sin),
                  slot_mapping, q_out, k_pages, v_pages, k_dense, v_dense, gate_out, tokens, heads, kv_heads, head_dim,
                  value_dim, page_size, rotary_dim, gates, bias};
    // Which kernel runs follows from the layer (no norm, no rotation, sizes in fours) and the engine's buffers alone.
    const bool alone = q_weight == nullptr && k_weight == nullptr && cos_sin == nullptr && splits <= MAX_UNROLLED_SPLITS &&
                       head_dim % 4 == 0 && value_dim % 4 == 0 && gates % 4 == 0 && row_width % 4 == 0 && split_stride % 4 == 0 &&
                       aligned16(qkv) && aligned16(bias) && aligned16(q_out) && aligned16(gate_out) &&
                       aligned16(k_pages) && aligned16(v_pages) && aligned16(k_dense) && aligned16(v_dense);
    if (alone) {
        const dim3 grid((row_width / 4 + 255) / 256, tokens);
        if (out_type == ME_BF16) return launch_kernel(qkv_bias_store_kernel<__nv_bfloat16>, grid, 256, 0, stream, a);
        return launch_kernel(qkv_bias_store_kernel<float>, grid, 256, 0, stream, a);
    }
    if (out_type == ME_BF16) {
        auto kernel = qk_wide_norm_rope_store_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_kernel(kernel, tokens, 256, smem, stream, a);
    }
    auto kernel = qk_wide_norm_rope_store_kernel<float>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_kernel(kernel, tokens, 256, smem, stream, a);
}

// ------------------------------------------------------ an activation on a product's partial sums

// out[t][i] = act(sum_s partial[s][t][i]) in the compute dtype, for a feed-forward without a gate.
// 0: relu(z)^2, 1: z * sigmoid(z), 2: the tanh form of GELU, 3: relu(z).
enum : int { ACT_RELU_SQUARED = 0, ACT_SILU = 1, ACT_GELU_TANH = 2, ACT_RELU = 3 };

__device__ __forceinline__ float plain_activation(float z, int activation) {
    if (activation == ACT_RELU_SQUARED) { const float r = fmaxf(z, 0.0f); return r * r; }
    if (activation == ACT_SILU) return z / (1.0f + expf(-z));
    if (activation == ACT_GELU_TANH) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    return fmaxf(z, 0.0f);
}

template <typename OutT, int V>  // V consecutive elements per thread: 4 (16-byte loads) or 1
__global__ void activation_kernel(const float* __restrict__ partial, int splits, size_t split_stride,
                                  OutT* __restrict__ out, size_t total, int activation) {
    pdl_trigger();
    pdl_wait();
    for (size_t idx = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) * V; idx < total;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x * V) {
        if constexpr (V == 4) {
            float4 z = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int s = 0; s < splits; ++s) add4(z, *reinterpret_cast<const float4*>(partial + s * split_stride + idx));
            store4(out + idx, make_float4(plain_activation(z.x, activation), plain_activation(z.y, activation),
                                          plain_activation(z.z, activation), plain_activation(z.w, activation)));
        } else {
            float z = 0.0f;
            for (int s = 0; s < splits; ++s) z += partial[s * split_stride + idx];
            out[idx] = from_float<OutT>(plain_activation(z, activation));
        }
    }
}

ME_EXPORT int me_activation(const float* partial, int splits, long long split_stride, void* out, int out_type,
                            int tokens, int width, int activation, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (activation < ACT_RELU_SQUARED || activation > ACT_RELU) return ME_ERR_ARGUMENT;
    const size_t total = static_cast<size_t>(tokens) * width;
    const bool vec = width % 4 == 0 && split_stride % 4 == 0 && aligned16(partial) && aligned16(out);
    const int threads = 256;
    const int blocks = static_cast<int>(std::min<size_t>((total / (vec ? 4 : 1) + threads - 1) / threads, 148 * 32));
    const size_t stride = static_cast<size_t>(split_stride);
    if (out_type == ME_BF16) {
        auto* o = static_cast<__nv_bfloat16*>(out);
        return vec ? launch_kernel(activation_kernel<__nv_bfloat16, 4>, blocks, threads, 0, stream, partial, splits, stride, o, total, activation)
                   : launch_kernel(activation_kernel<__nv_bfloat16, 1>, blocks, threads, 0, stream, partial, splits, stride, o, total, activation);
    }
    auto* o = static_cast<float*>(out);
    return vec ? launch_kernel(activation_kernel<float, 4>, blocks, threads, 0, stream, partial, splits, stride, o, total, activation)
               : launch_kernel(activation_kernel<float, 1>, blocks, threads, 0, stream, partial, splits, stride, o, total, activation);
}

// --------------------------------------- bias + rotary + unit norm behind the rotation + cache write

// One warp per (token, head) over the columns of qkv = [q heads | k heads | v heads]: the partial sums and the
// bias are added, the first rotary_dim elements of a q or k head are rotated (element e pairs with e +
// rotary_dim / 2), and then, with `unit_norm`, the rotated head is divided by its root mean square over head_dim
// (eps inside the root, no weight).  q goes to q_out, k and v to the token's cache slot (or to dense buffers).
// Lane l holds elements l, l + 32, ... and adds their squares in ascending order; the lanes meet in a butterfly.
struct UnitQkvArgs {
    const float* qkv;  // [splits][tokens][row_width]
    int splits;
    size_t split_stride;
    int row_width;
    const float* bias;      // [row_width] or null
    const float2* cos_sin;  // [tokens][rotary_dim / 2] or null
    const int* slot_mapping;
    void* q_out;
    void* k_pages;
    void* v_pages;
    void* k_dense;
    void* v_dense;
    float eps;
    int tokens, heads, kv_heads, head_dim, value_dim, page_size, rotary_dim, unit_norm;
};

constexpr int UNIT_WARPS = 4;
constexpr int UNIT_MAX_PER_LANE = 16;  // head sizes up to 512

template <typename OutT>
__global__ void __launch_bounds__(UNIT_WARPS * 32) qkv_rope_unit_store_kernel(UnitQkvArgs a) {
    extern __shared__ float staged[];  // [UNIT_WARPS][max(head_dim, value_dim)]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_token = a.heads + 2 * a.kv_heads;
    const long long item = static_cast<long long>(blockIdx.x) * UNIT_WARPS + warp;
    pdl_trigger();
    pdl_wait();
    if (item >= static_cast<long long>(a.tokens) * per_token) return;
    const int token = static_cast<int>(item / per_token), which = static_cast<int>(item % per_token);
    const int q_width = a.heads * a.head_dim, k_width = a.kv_heads * a.head_dim;
    const bool is_q = which < a.heads, is_k = !is_q && which < a.heads + a.kv_heads;
    const int head = is_q ? which : is_k ? which - a.heads : which - a.heads - a.kv_heads;
    const int d = (is_q || is_k) ? a.head_dim : a.value_dim;
    const int column = is_q ? head * d : is_k ? q_width + head * d : q_width + k_width + head * d;
    float* mine = staged + warp * max(a.head_dim, a.value_dim);
    const float* src = a.qkv + static_cast<size_t>(token) * a.row_width + column;
    for (int e = lane; e < d; e += 32) {
        float v = 0.0f;
        for (int s = 0; s < a.splits; ++s) v += src[s * a.split_stride + e];
        if (a.bias) v += a.bias[column + e];
        mine[e] = v;
    }
    __syncwarp();
    float value[UNIT_MAX_PER_LANE];
    float sum_sq = 0.0f;
    const int half = a.rotary_dim / 2;
    const float2* angles = (a.cos_sin && (is_q || is_k)) ? a.cos_sin + static_cast<size_t>(token) * half : nullptr;
#pragma unroll
    for (int j = 0; j < UNIT_MAX_PER_LANE; ++j) {
        const int e = lane + 32 * j;
        if (e >= d) break;
        float v = mine[e];
        if (angles && e < a.rotary_dim) {
            const float other = mine[e < half ? e + half : e - half];
            const float2 angle = angles[e < half ? e : e - half];
            v = e < half ? v * angle.x - other * angle.y : v * angle.x + other * angle.y;
        }
        value[j] = v;
        sum_sq = fmaf(v, v, sum_sq);
    }
    float inv = 1.0f;
    if (a.unit_norm && (is_q || is_k)) inv = rsqrtf(warp_sum(sum_sq) / static_cast<float>(d) + a.eps);
    OutT* dst;
    if (is_q) {
        dst = static_cast<OutT*>(a.q_out) + static_cast<size_t>(token) * q_width + column;
    } else if (a.slot_mapping) {
        const int slot = a.slot_mapping[token];
        if (slot < 0) return;
        const size_t page = slot / a.page_size, offset = slot % a.page_size;
        dst = static_cast<OutT*>(is_k ? a.k_pages : a.v_pages) + ((page * a.kv_heads + head) * a.page_size + offset) * d;
    } else {
        dst = static_cast<OutT*>(is_k ? a.k_dense : a.v_dense) + static_cast<size_t>(token) * a.kv_heads * d + head * d;
    }
#pragma unroll
    for (int j = 0; j < UNIT_MAX_PER_LANE; ++j) {
        const int e = lane + 32 * j;
        if (e >= d) break;
        dst[e] = from_float<OutT>(value[j] * inv);
    }
}

ME_EXPORT int me_qkv_rope_unit_store(const float* qkv, int splits, long long split_stride, int row_width,
                                     const float* bias, const float* cos_sin, const int* slot_mapping, void* q_out,
                                     void* k_pages, void* v_pages, void* k_dense, void* v_dense, float eps, int out_type,
                                     int tokens, int heads, int kv_heads, int head_dim, int value_dim, int page_size,
                                     int rotary_dim, int unit_norm, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > head_dim || rotary_dim % 2) return ME_ERR_ARGUMENT;
    if (row_width < (heads + kv_heads) * head_dim + kv_heads * value_dim) return ME_ERR_ARGUMENT;
    if (head_dim < 1 || value_dim < 1 || head_dim > 32 * UNIT_MAX_PER_LANE || value_dim > 32 * UNIT_MAX_PER_LANE)
        return ME_ERR_UNSUPPORTED;
    UnitQkvArgs a{qkv, splits, (size_t)split_stride, row_width, bias, reinterpret_cast<const float2*>(cos_sin), slot_mapping,
                  q_out, k_pages, v_pages, k_dense, v_dense, eps, tokens, heads, kv_heads, head_dim, value_dim, page_size,
                  rotary_dim, unit_norm};
    const long long items = static_cast<long long>(tokens) * (heads + 2 * kv_heads);
    const int blocks = static_cast<int>((items + UNIT_WARPS - 1) / UNIT_WARPS);
    const size_t smem = static_cast<size_t>(UNIT_WARPS) * std::max(head_dim, value_dim) * sizeof(float);
    if (out_type == ME_BF16) return launch_kernel(qkv_rope_unit_store_kernel<__nv_bfloat16>, blocks, UNIT_WARPS * 32, smem, stream, a);
    return launch_kernel(qkv_rope_unit_store_kernel<float>, blocks, UNIT_WARPS * 32, smem, stream, a);
}
