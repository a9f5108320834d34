// Several residual streams per token ("hyper-connections"): a sublayer reads a weighted sum of the streams, and
// its output enters every stream with a share of its own while the streams are mixed among themselves.
//
//   u       = sum_s read[s] x_s                                  what the sublayer's norm sees
//   x_t new = sum_s mix[s][t] x_s + (mult * share[t]) * y        all streams at once, from the old ones
//
// One kernel does, for one row: the update that the *previous* sublayer's output y (partial sums of a split
// product, added in ascending order) is still owed, the write-back of the new streams, the read for the *next*
// sublayer, and that sublayer's RMS norm: out = weight * u * rsqrt(mean(u^2) + eps).  Everything is float32.
//
//   seed     non-null: the streams have not been written yet and every one of them equals this row array (the
//            embedding's output); the new streams are written from it.
//   pending  null: no update is owed (the first sublayer of a model); the streams are then left alone.
//   read     null: u is the plain sum of the streams (the model's end).
//   rows     non-null: only the listed rows are produced and nothing is written back.
//
// One block per output row.  Column i's square goes to the partial sum of thread (i / V) % 256 in ascending
// order, the lanes of a warp meet in a butterfly and the warps in ascending order: a row's statistics are the
// same bits whatever else is in the batch.
#include "common.cuh"

#include <algorithm>

constexpr int MAX_STREAMS = 8;
constexpr int HYPER_THREADS = 256;

struct HyperArgs {
    float* streams;  // [count][tokens][hidden]
    size_t stream_stride;
    const float* seed;     // [tokens][hidden] or null
    const float* pending;  // [splits][tokens][hidden] or null
    int splits;
    size_t split_stride;
    const float* mix;    // [count][count], [from][to]
    const float* share;  // [count]
    float mult;
    const float* read;    // [count] or null
    const float* weight;  // [hidden]
    float eps;
    void* out;        // [rows][hidden]
    const int* rows;  // or null
    int hidden, count;
};

__device__ __forceinline__ void store_out(float* dst, float v) { *dst = v; }
__device__ __forceinline__ void store_out(__nv_bfloat16* dst, float v) { *dst = __float2bfloat16_rn(v); }

template <typename OutT, int V>  // V consecutive columns per thread: 4 (16-byte accesses) or 1
__global__ void __launch_bounds__(HYPER_THREADS) hyper_step_kernel(HyperArgs a) {
    extern __shared__ float row_cache[];  // [hidden]
    __shared__ float warp_partial[HYPER_THREADS / 32];
    __shared__ float coefficient[MAX_STREAMS * MAX_STREAMS + 2 * MAX_STREAMS];
    const int out_row = blockIdx.x;
    const int count = a.count;
    float* mix = coefficient;
    float* share = coefficient + MAX_STREAMS * MAX_STREAMS;
    float* read = share + MAX_STREAMS;
    pdl_trigger();
    // The layer's coefficients are weights: fetched ahead of the wait.
    const bool update = a.pending != nullptr;
    for (int i = threadIdx.x; i < count * count; i += HYPER_THREADS) mix[i] = update ? a.mix[i] : 0.0f;
    for (int i = threadIdx.x; i < count; i += HYPER_THREADS) {
        share[i] = update ? a.mult * a.share[i] : 0.0f;
        read[i] = a.read ? a.read[i] : 1.0f;
    }
    const int src = a.rows ? a.rows[out_row] : out_row;
    __syncthreads();
    pdl_wait();
    const size_t row_offset = static_cast<size_t>(src) * a.hidden;
    const bool write_back = a.rows == nullptr && update;
    float sum_sq = 0.0f;
    for (int i = threadIdx.x * V; i < a.hidden; i += HYPER_THREADS * V) {
        float old[MAX_STREAMS][V];
        if (a.seed != nullptr) {
            float first[V];
            if constexpr (V == 4) {
                const float4 v = *reinterpret_cast<const float4*>(a.seed + row_offset + i);
                first[0] = v.x, first[1] = v.y, first[2] = v.z, first[3] = v.w;
            } else {
                first[0] = a.seed[row_offset + i];
            }
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s)
#pragma unroll
                for (int v = 0; v < V; ++v) old[s][v] = first[v];
        } else {
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s) {
                if (s >= count) continue;
                const float* p = a.streams + s * a.stream_stride + row_offset + i;
                if constexpr (V == 4) {
                    const float4 v = *reinterpret_cast<const float4*>(p);
                    old[s][0] = v.x, old[s][1] = v.y, old[s][2] = v.z, old[s][3] = v.w;
                } else {
                    old[s][0] = *p;
                }
            }
        }
        float u[V];
#pragma unroll
        for (int v = 0; v < V; ++v) u[v] = 0.0f;
        if (update) {
            float y[V];
#pragma unroll
            for (int v = 0; v < V; ++v) y[v] = 0.0f;
            for (int s = 0; s < a.splits; ++s) {
                const float* p = a.pending + s * a.split_stride + row_offset + i;
                if constexpr (V == 4) {
                    const float4 v = *reinterpret_cast<const float4*>(p);
                    y[0] += v.x, y[1] += v.y, y[2] += v.z, y[3] += v.w;
                } else {
                    y[0] += *p;
                }
            }
#pragma unroll
            for (int t = 0; t < MAX_STREAMS; ++t) {
                if (t >= count) continue;
                float fresh[V];
#pragma unroll
                for (int v = 0; v < V; ++v) fresh[v] = 0.0f;
#pragma unroll
                for (int s = 0; s < MAX_STREAMS; ++s) {
                    if (s >= count) continue;
                    const float c = mix[s * count + t];
#pragma unroll
                    for (int v = 0; v < V; ++v) fresh[v] = fmaf(c, old[s][v], fresh[v]);
                }
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    fresh[v] = fmaf(share[t], y[v], fresh[v]);
                    u[v] = fmaf(read[t], fresh[v], u[v]);
                }
                if (write_back) {
                    float* p = a.streams + t * a.stream_stride + row_offset + i;
                    if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(fresh[0], fresh[1], fresh[2], fresh[3]);
                    else *p = fresh[0];
                }
            }
        } else {
#pragma unroll
            for (int t = 0; t < MAX_STREAMS; ++t) {
                if (t >= count) continue;
#pragma unroll
                for (int v = 0; v < V; ++v) u[v] = fmaf(read[t], old[t][v], u[v]);
            }
        }
#pragma unroll
        for (int v = 0; v < V; ++v) {
            row_cache[i + v] = u[v];
            sum_sq = fmaf(u[v], u[v], sum_sq);
        }
    }
    sum_sq = warp_sum(sum_sq);
    if ((threadIdx.x & 31) == 0) warp_partial[threadIdx.x >> 5] = sum_sq;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < HYPER_THREADS / 32; ++w) total += warp_partial[w];
    const float inv = rsqrtf(total / static_cast<float>(a.hidden) + a.eps);
    OutT* out = static_cast<OutT*>(a.out) + static_cast<size_t>(out_row) * a.hidden;
    for (int i = threadIdx.x; i < a.hidden; i += HYPER_THREADS) store_out(out + i, a.weight[i] * (row_cache[i] * inv));
}

static bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

ME_EXPORT int me_hyper_step(float* streams, long long stream_stride, const float* seed, const float* pending,
                            int splits, long long split_stride, const float* mix, const float* share, float mult,
                            const float* read, const float* weight, float eps, void* out, int out_type,
                            const int* rows, int count_rows, int hidden, int count, cudaStream_t stream) {
    if (count_rows <= 0) return 0;
    if (count < 1 || count > MAX_STREAMS) return ME_ERR_UNSUPPORTED;
    if (pending != nullptr && (mix == nullptr || share == nullptr || splits < 1)) return ME_ERR_ARGUMENT;
    const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
    if (smem > 200 * 1024) return ME_ERR_UNSUPPORTED;
    HyperArgs a{streams, static_cast<size_t>(stream_stride), seed, pending, splits, static_cast<size_t>(split_stride),
                mix, share, mult, read, weight, eps, out, rows, hidden, count};
    // Which form runs follows from the width and the engine's buffers alone; both give a column the same bits.
    const bool vec = hidden % 4 == 0 && stream_stride % 4 == 0 && split_stride % 4 == 0 && aligned16(streams) &&
                     aligned16(seed) && aligned16(pending);
    auto launch = [&](auto kernel) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_kernel(kernel, count_rows, HYPER_THREADS, smem, stream, a);
    };
    if (out_type == ME_BF16) return vec ? launch(hyper_step_kernel<__nv_bfloat16, 4>) : launch(hyper_step_kernel<__nv_bfloat16, 1>);
    return vec ? launch(hyper_step_kernel<float, 4>) : launch(hyper_step_kernel<float, 1>);
}

// sum[t][i] = sum_s x_s[t][i] after the update that `pending` is owed (see above), float32: the streams as one
// residual row array, for whoever wants to look at it between layers.  Nothing is written back.
__global__ void __launch_bounds__(256) hyper_sum_kernel(HyperArgs a, float* __restrict__ sum, size_t total) {
    pdl_trigger();
    pdl_wait();
    const bool update = a.pending != nullptr;
    for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float old[MAX_STREAMS];
        for (int s = 0; s < a.count; ++s) old[s] = a.seed ? a.seed[idx] : a.streams[s * a.stream_stride + idx];
        float y = 0.0f;
        for (int s = 0; s < (update ? a.splits : 0); ++s) y += a.pending[s * a.split_stride + idx];
        float u = 0.0f;
        for (int t = 0; t < a.count; ++t) {
            float fresh = old[t];
            if (update) {
                fresh = 0.0f;
                for (int s = 0; s < a.count; ++s) fresh = fmaf(a.mix[s * a.count + t], old[s], fresh);
                fresh = fmaf(a.mult * a.share[t], y, fresh);
            }
            u += fresh;
        }
        sum[idx] = u;
    }
}

ME_EXPORT int me_hyper_sum(const float* streams, long long stream_stride, const float* seed, const float* pending,
                           int splits, long long split_stride, const float* mix, const float* share, float mult,
                           float* sum, int tokens, int hidden, int count, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (count < 1 || count > MAX_STREAMS) return ME_ERR_UNSUPPORTED;
    HyperArgs a{const_cast<float*>(streams), static_cast<size_t>(stream_stride), seed, pending, splits,
                static_cast<size_t>(split_stride), mix, share, mult, nullptr, nullptr, 0.0f, nullptr, nullptr, hidden, count};
    const size_t total = static_cast<size_t>(tokens) * hidden;
    const int blocks = static_cast<int>(std::min<size_t>((total + 255) / 256, 148 * 16));
    return launch_kernel(hyper_sum_kernel, blocks, 256, 0, stream, a, sum, total);
}
