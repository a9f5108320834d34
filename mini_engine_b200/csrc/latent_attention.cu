// Kernels of attention through a low-rank latent: keys and values of all heads are linear maps of one cached
// vector c per token (plus one rotated key part that all heads share), so the maps are applied to the query and
// to the attention's output instead of to every cached token:
//
//   score_h(i, j) = q_plain_h(i) . (U_k,h c_j) + q_rot_h(i) . k_rot(j)  =  [U_k,h^T q_plain_h(i) | q_rot_h(i)] . [c_j | k_rot(j)]
//   out_h(i)      = sum_j p_h(i, j) U_v,h c_j                            =  U_v,h (sum_j p_h(i, j) c_j)
//
// The cache holds one row [c | k_rot] per token; attention runs as one shared key/value head whose values are
// the first `rank` elements of its keys.  Three kernels around it:
//
//   latent_down_finish   the row [q latent | c | k_rot | gates] of the fused down projection: RMS norm of the
//                        query latent and of c (each with its weight), rotation of k_rot, the cache write, and
//                        sigmoid of the gates; statistics, angles and gates in float32.
//   head_product         out[t][h][n] = sum_k in[t][h][k] W[h][k][n] for every head, one accumulator per output
//                        in ascending k (a token's bits never depend on the batch); used for U_k^T q and for
//                        U_v o.  `tail` more input columns per head are rotated and appended to the output (the
//                        rotated query part).
#include "common.cuh"

// ------------------------------------------------------------------- down projection's finish

struct DownArgs {
    const float* down;  // [splits][tokens][row_width]: q latent (q_rank, may be 0) | c (kv_rank) | k_rot (rot_dim) | gates
    int splits;
    size_t split_stride;
    int row_width;
    const float* q_weight;   // [q_rank]
    const float* kv_weight;  // [kv_rank]
    float eps;
    const float2* cos_sin;  // [tokens][rotary_dim / 2] or null
    const int* slot_mapping;
    void* q_latent_out;  // [tokens][q_rank]
    void* k_pages;       // rows of kv_rank + rot_dim, one per slot
    float* gate_out;     // [tokens][gates]
    int tokens, q_rank, kv_rank, rot_dim, rotary_dim, gates;
};

template <typename OutT>
__global__ void __launch_bounds__(256) latent_down_finish_kernel(DownArgs a) {
    extern __shared__ float row[];  // [row_width]
    __shared__ float warp_partial[2][8];
    const int token = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_trigger();
    pdl_wait();
    const float* src = a.down + static_cast<size_t>(token) * a.row_width;
    float q_sq = 0.0f, c_sq = 0.0f;
    for (int i = threadIdx.x; i < a.row_width; i += 256) {
        float v = 0.0f;
        if (a.splits <= 8) {  // all loads of the column first, then the sum in the same ascending order
            float part[8];
#pragma unroll
            for (int s = 0; s < 8; ++s)
                if (s < a.splits) part[s] = src[s * a.split_stride + i];
#pragma unroll
            for (int s = 0; s < 8; ++s)
                if (s < a.splits) v += part[s];
        } else {
            for (int s = 0; s < a.splits; ++s) v += src[s * a.split_stride + i];
        }
        row[i] = v;
        if (i < a.q_rank) q_sq = fmaf(v, v, q_sq);
        else if (i < a.q_rank + a.kv_rank) c_sq = fmaf(v, v, c_sq);
    }
    q_sq = warp_sum(q_sq), c_sq = warp_sum(c_sq);
    if (lane == 0) warp_partial[0][warp] = q_sq, warp_partial[1][warp] = c_sq;
    __syncthreads();
    float q_total = 0.0f, c_total = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) q_total += warp_partial[0][w], c_total += warp_partial[1][w];
    const float q_inv = a.q_rank > 0 ? rsqrtf(q_total / static_cast<float>(a.q_rank) + a.eps) : 1.0f;  // no query latent: nothing to norm
    const float c_inv = rsqrtf(c_total / static_cast<float>(a.kv_rank) + a.eps);
    const int half = a.rotary_dim / 2;
    const float2* angles = a.cos_sin ? a.cos_sin + static_cast<size_t>(token) * half : nullptr;
    const int slot = a.slot_mapping[token];
    const int key_width = a.kv_rank + a.rot_dim;
    OutT* key_row = slot >= 0 ? static_cast<OutT*>(a.k_pages) + static_cast<size_t>(slot) * key_width : nullptr;
    for (int i = threadIdx.x; i < a.row_width; i += 256) {
        if (i < a.q_rank) {
            static_cast<OutT*>(a.q_latent_out)[static_cast<size_t>(token) * a.q_rank + i] =
                from_float<OutT>(row[i] * q_inv * a.q_weight[i]);
        } else if (i < a.q_rank + a.kv_rank) {
            const int e = i - a.q_rank;
            if (key_row) key_row[e] = from_float<OutT>(row[i] * c_inv * a.kv_weight[e]);
        } else if (i < a.q_rank + key_width) {
            const int e = i - a.q_rank - a.kv_rank;
            float value = row[i];
            if (angles && e < a.rotary_dim) {
                const float other = row[e < half ? i + half : i - half];
                const float2 angle = angles[e < half ? e : e - half];
                value = e < half ? value * angle.x - other * angle.y : value * angle.x + other * angle.y;
            }
            if (key_row) key_row[a.kv_rank + e] = from_float<OutT>(value);
        } else {
            const int g = i - a.q_rank - key_width;
            if (g < a.gates) a.gate_out[static_cast<size_t>(token) * a.gates + g] = 1.0f / (1.0f + expf(-row[i]));
        }
    }
}

ME_EXPORT int me_latent_down_finish(const float* down, int splits, long long split_stride, int row_width,
                                    const float* q_weight, const float* kv_weight, float eps, const float* cos_sin,
                                    const int* slot_mapping, void* q_latent_out, void* k_pages, float* gate_out,
                                    int out_type, int tokens, int q_rank, int kv_rank, int rot_dim, int rotary_dim,
                                    int gates, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > rot_dim || rotary_dim % 2) return ME_ERR_ARGUMENT;
    if (row_width < q_rank + kv_rank + rot_dim + gates || q_rank < 0 || kv_rank < 1) return ME_ERR_ARGUMENT;
    if (gates > 0 && gate_out == nullptr) return ME_ERR_ARGUMENT;
    const size_t smem = static_cast<size_t>(row_width) * sizeof(float);
    if (smem > 200 * 1024) return ME_ERR_UNSUPPORTED;
    DownArgs a{down, splits, (size_t)split_stride, row_width, q_weight, kv_weight, eps,
               reinterpret_cast<const float2*>(cos_sin), slot_mapping, q_latent_out, k_pages, gate_out,
               tokens, q_rank, kv_rank, rot_dim, rotary_dim, gates};
    if (out_type == ME_BF16) {
        auto kernel = latent_down_finish_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_kernel(kernel, tokens, 256, smem, stream, a);
    }
    auto kernel = latent_down_finish_kernel<float>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_kernel(kernel, tokens, 256, smem, stream, a);
}

// ------------------------------------------------------------------------ products per head

constexpr int HP_TOKENS = 8;  // tokens that share one pass over a head's matrix

struct HeadProductArgs {
    const void* in;  // [splits][tokens][heads * in_head] (float partial sums) or [tokens][heads * in_head] (InT)
    int splits;
    size_t split_stride;
    const void* weight;     // [heads][inner][outs]
    const float2* cos_sin;  // [tokens][rotary_dim / 2] or null
    void* out;              // [tokens][heads][outs + tail]
    int tokens, heads, inner, outs, tail, rotary_dim;
};

template <typename InT, typename T>
__global__ void __launch_bounds__(128) head_product_kernel(HeadProductArgs a) {
    extern __shared__ float staged[];  // [HP_TOKENS][inner + tail]
    const int head = blockIdx.y, first = blockIdx.x * HP_TOKENS;
    const int count = min(HP_TOKENS, a.tokens - first);
    const int in_head = a.inner + a.tail, out_head = a.outs + a.tail;
    pdl_trigger();
    pdl_wait();
    const InT* in = static_cast<const InT*>(a.in);
    for (int i = threadIdx.x; i < HP_TOKENS * in_head; i += 128) {
        const int t = i / in_head, k = i % in_head;
        float v = 0.0f;
        if (t < count) {
            const size_t at = (static_cast<size_t>(first + t) * a.heads + head) * in_head + k;
            for (int s = 0; s < a.splits; ++s) v += to_float(in[s * a.split_stride + at]);
        }
        staged[i] = v;
    }
    __syncthreads();
    const T* weight = static_cast<const T*>(a.weight) + static_cast<size_t>(head) * a.inner * a.outs;
    T* out = static_cast<T*>(a.out);
    for (int n = threadIdx.x; n < a.outs; n += 128) {
        float acc[HP_TOKENS];
#pragma unroll
        for (int t = 0; t < HP_TOKENS; ++t) acc[t] = 0.0f;
        for (int k = 0; k < a.inner; ++k) {
            const float w = to_float(weight[static_cast<size_t>(k) * a.outs + n]);
#pragma unroll
            for (int t = 0; t < HP_TOKENS; ++t) acc[t] = fmaf(staged[t * in_head + k], w, acc[t]);
        }
#pragma unroll
        for (int t = 0; t < HP_TOKENS; ++t)
            if (t < count) out[(static_cast<size_t>(first + t) * a.heads + head) * out_head + n] = from_float<T>(acc[t]);
    }
    const int half = a.rotary_dim / 2;
    for (int i = threadIdx.x; i < count * a.tail; i += 128) {
        const int t = i / a.tail, e = i % a.tail;
        const float* part = staged + t * in_head + a.inner;
        float value = part[e];
        if (a.cos_sin && e < a.rotary_dim) {
            const float other = part[e < half ? e + half : e - half];
            const float2 angle = a.cos_sin[static_cast<size_t>(first + t) * half + (e < half ? e : e - half)];
            value = e < half ? value * angle.x - other * angle.y : value * angle.x + other * angle.y;
        }
        out[(static_cast<size_t>(first + t) * a.heads + head) * out_head + a.outs + e] = from_float<T>(value);
    }
}

// in_type: ME_F32 for float input (partial sums allowed), else the input has the type of the weights and output.
ME_EXPORT int me_head_product(const void* in, int in_type, int splits, long long split_stride, const void* weight,
                              const float* cos_sin, void* out, int type, int tokens, int heads, int inner, int outs,
                              int tail, int rotary_dim, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (heads < 1 || inner < 1 || outs < 1 || tail < 0 || rotary_dim < 0 || rotary_dim > tail || rotary_dim % 2)
        return ME_ERR_ARGUMENT;
    if (in_type != ME_F32 && (in_type != type || splits != 1)) return ME_ERR_ARGUMENT;
    const size_t smem = static_cast<size_t>(HP_TOKENS) * (inner + tail) * sizeof(float);
    if (smem > 200 * 1024) return ME_ERR_UNSUPPORTED;
    HeadProductArgs a{in, splits, (size_t)split_stride, weight, reinterpret_cast<const float2*>(cos_sin), out,
                      tokens, heads, inner, outs, tail, rotary_dim};
    const dim3 grid((tokens + HP_TOKENS - 1) / HP_TOKENS, heads);
#define ME_LAUNCH_HEAD_PRODUCT(IN, T)                                                                              \
    {                                                                                                              \
        auto kernel = head_product_kernel<IN, T>;                                                                  \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return launch_kernel(kernel, grid, 128, smem, stream, a);                                                  \
    }
    if (type == ME_BF16) {
        if (in_type == ME_F32) ME_LAUNCH_HEAD_PRODUCT(float, __nv_bfloat16)
        ME_LAUNCH_HEAD_PRODUCT(__nv_bfloat16, __nv_bfloat16)
    }
    ME_LAUNCH_HEAD_PRODUCT(float, float)
#undef ME_LAUNCH_HEAD_PRODUCT
}
