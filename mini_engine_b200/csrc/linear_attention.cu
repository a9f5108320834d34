// Gated linear attention: a per-head matrix state with a decay per key channel.
//
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,   S: [dim][vdim] per head, float32,
//   alpha_t = sigmoid(z_t)^(1/tau),  z_t = A2 (A1 h_t) + b  (a low-rank projection of the layer's input),
//
// then every head's o_t is divided by its root mean square over vdim (eps inside the root), multiplied by
// a weight [vdim] shared by the heads and by silu of a gate projection, and leaves in the compute dtype
// for the output projection.  The state of a request lives in its slot of the cache manager's state
// array between steps; an entry that starts at position 0 starts from zero.
//
// Prepare kernel: for all tokens at once, the sum of the product's partial sums, the query scale and the
// decay from the low-rank sums, in 32-bit.  Scan kernel: one warp per (entry, head, 32 value columns).  Each
// lane owns one column of the state in registers ([dim] floats) and walks the entry's tokens in order, so
// the serial part is two multiply-adds per state element and token.  Columns are independent, hence the result does not depend on how the work is cut
// over warps, and a token's output depends on the tokens before it only through the state: the bits are
// the same for a whole prompt, its portions and single decoded tokens.
//
// Finish kernel: one warp per (token, head): unit norm, weight, gate.
#include "common.cuh"

#include <algorithm>

// log(sigmoid(z)) without overflow: -softplus(-z).
__device__ __forceinline__ float log_sigmoid(float z) {
    return z >= 0.0f ? -log1pf(expf(-z)) : z - log1pf(expf(z));
}

// ------------------------------------------------------------------------------- prepare

// For every token, head and key channel: q (scaled), k and the decay, float32, as
// prepared[token][head][0..2][dim].  A block takes PREP_TOKENS tokens, so that a row of the decay's
// second factor (stored transposed, [rank][heads*dim]) is read once for all of them.
struct PrepArgs {
    const float* proj;  // [splits][tokens][width] partial sums of the fused input projection
    int splits;
    size_t split_stride;
    int width;
    int q_col, k_col, a_col;  // first column of q [heads*dim], k [heads*dim], low-rank sums [rank]
    const float* a2t;         // [rank][heads*dim]
    const float* a2_bias;     // [heads*dim]
    float* prepared;          // [tokens][heads][3][dim]
    float q_scale, inv_tau;
    int tokens, heads, dim, rank;
};

constexpr int PREP_TOKENS = 8;

__global__ void __launch_bounds__(256) gla_prepare_kernel(PrepArgs a) {
    extern __shared__ float low[];  // [PREP_TOKENS][rank]
    const int first = blockIdx.x * PREP_TOKENS;
    const int count = min(PREP_TOKENS, a.tokens - first);
    pdl_trigger();
    pdl_wait();
    for (int i = threadIdx.x; i < count * a.rank; i += blockDim.x) {
        const int t = i / a.rank, r = i % a.rank;
        const float* src = a.proj + static_cast<size_t>(first + t) * a.width + a.a_col + r;
        float sum = 0.0f;
        for (int p = 0; p < a.splits; ++p) sum += src[p * a.split_stride];
        low[i] = sum;
    }
    __syncthreads();
    const int items = a.heads * a.dim;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < items; i += gridDim.y * blockDim.x) {
        float z[PREP_TOKENS];
#pragma unroll
        for (int t = 0; t < PREP_TOKENS; ++t) z[t] = 0.0f;
        for (int r = 0; r < a.rank; ++r) {
            const float w = a.a2t[static_cast<size_t>(r) * items + i];
#pragma unroll
            for (int t = 0; t < PREP_TOKENS; ++t)
                if (t < count) z[t] = fmaf(w, low[t * a.rank + r], z[t]);
        }
        const float bias = a.a2_bias[i];
        const int head = i / a.dim, d = i % a.dim;
#pragma unroll
        for (int t = 0; t < PREP_TOKENS; ++t) {
            if (t >= count) break;
            const float* row = a.proj + static_cast<size_t>(first + t) * a.width + i;
            float q = 0.0f, k = 0.0f;
            for (int p = 0; p < a.splits; ++p) {
                q += row[p * a.split_stride + a.q_col];
                k += row[p * a.split_stride + a.k_col];
            }
            float* dst = a.prepared + ((static_cast<size_t>(first + t) * a.heads + head) * 3) * a.dim + d;
            dst[0] = q * a.q_scale;
            dst[a.dim] = k;
            dst[2 * a.dim] = expf(log_sigmoid(z[t] + bias) * a.inv_tau);
        }
    }
}

// ---------------------------------------------------------------------------------- scan

struct ScanArgs {
    const float* proj;  // [splits][tokens][width]: the value columns are read from here
    int splits;
    size_t split_stride;
    int width;
    int v_col;               // first column of v [heads*vdim]
    const float* prepared;   // [tokens][heads][3][dim] from the prepare kernel
    const int* cu_tokens;    // [entries + 1]
    const int* state_slots;  // [entries]
    const int* fresh;        // [entries] 1: the entry starts its request, the state starts at zero
    float* state;            // [slots + 1][heads][dim][vdim]
    float* out;              // [tokens][heads][vdim] float32: o_t before the norm
    int heads, dim, vdim;
    int max_count = 0;       // > 0: entries with more tokens than this are left to the chunked kernels
};

constexpr int SCAN_CHUNK = 16;

__device__ __forceinline__ void copy_async_16(float* shared_dst, const float* global_src) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(shared_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(global_src) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int LEFT>
__device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(LEFT) : "memory"); }

// One warp per (entry, head, 32 value columns); a lane keeps its column of the state in registers.
// q, k and decay of the next chunk of tokens arrive in shared memory (asynchronous copies, two buffers)
// and its values in registers while the current chunk is computed.
template <int DIMP>  // dim rounded up: the registers a lane holds of its state column
__global__ void __launch_bounds__(32) gla_scan_kernel(ScanArgs a) {
    extern __shared__ __align__(16) float staged[];
    constexpr int TILE = SCAN_CHUNK * 3 * DIMP;
    float* tiles = staged;              // [2][SCAN_CHUNK][3][DIMP]
    float* v_s = staged + 2 * TILE;     // [2][SCAN_CHUNK][32] this warp's value columns
    const int entry = blockIdx.x, head = blockIdx.y, lane = threadIdx.x;
    const int column = blockIdx.z * 32 + lane;
    const bool live = column < a.vdim;
    const int dim = a.dim;
    const bool vector = dim % 4 == 0;
    for (int i = lane; i < 2 * SCAN_CHUNK * 3 * (DIMP - dim); i += 32)  // channels dim..DIMP are zero for good
        tiles[(i / (DIMP - dim)) * DIMP + dim + i % (DIMP - dim)] = 0.0f;
    __syncwarp();
    pdl_trigger();
    pdl_wait();
    const int begin = a.cu_tokens[entry], end = a.cu_tokens[entry + 1];
    if (a.max_count > 0 && end - begin > a.max_count) return;
    float* state = a.state + ((static_cast<size_t>(a.state_slots[entry]) * a.heads + head) * dim) * a.vdim + column;

    float s[DIMP];
    const bool from_zero = a.fresh[entry] != 0;
#pragma unroll
    for (int d = 0; d < DIMP; ++d) s[d] = (live && !from_zero && d < dim) ? state[static_cast<size_t>(d) * a.vdim] : 0.0f;

    auto stage_tile = [&](int chunk, int buffer) {  // q, k, decay of tokens chunk .. chunk + count
        const int count = min(SCAN_CHUNK, end - chunk);
        float* tile = tiles + buffer * TILE;
        if (vector) {
            const int quads = 3 * dim / 4;
            for (int i = lane; i < count * quads; i += 32) {
                const int t = i / quads, j = (i % quads) * 4;
                const int which = j / dim, d = j % dim;
                copy_async_16(tile + (t * 3 + which) * DIMP + d,
                              a.prepared + ((static_cast<size_t>(chunk + t) * a.heads + head) * 3) * dim + j);
            }
        } else {
            for (int i = lane; i < count * 3 * dim; i += 32) {
                const int t = i / (3 * dim), j = i % (3 * dim);
                tile[(t * 3 + j / dim) * DIMP + j % dim] = a.prepared[((static_cast<size_t>(chunk + t) * a.heads + head) * 3) * dim + j];
            }
        }
        copy_async_commit();
    };
    auto load_values = [&](int chunk, float (&v)[SCAN_CHUNK]) {
        const int count = min(SCAN_CHUNK, end - chunk);
#pragma unroll
        for (int t = 0; t < SCAN_CHUNK; ++t) {
            v[t] = 0.0f;
            if (live && t < count) {
                const float* src = a.proj + static_cast<size_t>(chunk + t) * a.width + a.v_col + head * a.vdim + column;
                for (int p = 0; p < a.splits; ++p) v[t] += src[p * a.split_stride];
            }
        }
    };

    float v_next[SCAN_CHUNK];
    if (begin < end) {
        stage_tile(begin, 0);
        load_values(begin, v_next);
#pragma unroll
        for (int t = 0; t < SCAN_CHUNK; ++t) v_s[t * 32 + lane] = v_next[t];
    }
    int buffer = 0;
    for (int chunk = begin; chunk < end; chunk += SCAN_CHUNK, buffer ^= 1) {
        const int count = min(SCAN_CHUNK, end - chunk);
        const bool more = chunk + SCAN_CHUNK < end;
        if (more) {
            stage_tile(chunk + SCAN_CHUNK, buffer ^ 1);
            load_values(chunk + SCAN_CHUNK, v_next);
            copy_async_wait<1>();
        } else {
            copy_async_wait<0>();
        }
        __syncwarp();
        const float* tile = tiles + buffer * TILE;
        const float* values = v_s + buffer * SCAN_CHUNK * 32;
#pragma unroll 1
        for (int t = 0; t < count; ++t) {
            const float v = values[t * 32 + lane];
            const float4* q4 = reinterpret_cast<const float4*>(tile + (t * 3 + 0) * DIMP);
            const float4* k4 = reinterpret_cast<const float4*>(tile + (t * 3 + 1) * DIMP);
            const float4* d4 = reinterpret_cast<const float4*>(tile + (t * 3 + 2) * DIMP);
            float o = 0.0f;
#pragma unroll
            for (int d = 0; d < DIMP; d += 4) {
                const float4 qq = q4[d / 4], kk = k4[d / 4], dd = d4[d / 4];
                s[d + 0] = fmaf(dd.x, s[d + 0], kk.x * v);
                s[d + 1] = fmaf(dd.y, s[d + 1], kk.y * v);
                s[d + 2] = fmaf(dd.z, s[d + 2], kk.z * v);
                s[d + 3] = fmaf(dd.w, s[d + 3], kk.w * v);
                o = fmaf(s[d + 0], qq.x, o);
                o = fmaf(s[d + 1], qq.y, o);
                o = fmaf(s[d + 2], qq.z, o);
                o = fmaf(s[d + 3], qq.w, o);
            }
            if (live) a.out[(static_cast<size_t>(chunk + t) * a.heads + head) * a.vdim + column] = o;
        }
        __syncwarp();
        if (more) {
#pragma unroll
            for (int t = 0; t < SCAN_CHUNK; ++t) v_s[(buffer ^ 1) * SCAN_CHUNK * 32 + t * 32 + lane] = v_next[t];
        }
    }
    if (live) {
#pragma unroll
        for (int d = 0; d < DIMP; ++d)
            if (d < dim) state[static_cast<size_t>(d) * a.vdim] = s[d];
    }
}

template <int DIMP>
static int launch_scan(const ScanArgs& a, int entries, cudaStream_t stream) {
    static SharedMemoryOptIn opt_in;
    const size_t smem = (static_cast<size_t>(2) * SCAN_CHUNK * (3 * DIMP + 32)) * sizeof(float);
    if (smem > 200 * 1024) return ME_ERR_UNSUPPORTED;
    if (smem > 48 * 1024) {
        const int code = opt_in(gla_scan_kernel<DIMP>, static_cast<int>(smem));
        if (code) return code;
    }
    const dim3 grid(entries, a.heads, (a.vdim + 31) / 32);
    return launch_kernel_in_order(gla_scan_kernel<DIMP>, grid, 32, smem, stream, a);
}

// Both kernels, one after the other: `prepared` is scratch of tokens * heads * 3 * dim floats, `a2t` the
// decay's second factor transposed to [rank][heads*dim].
ME_EXPORT int me_gla_scan(const float* proj, int splits, long long split_stride, int width, int q_col, int k_col,
                          int v_col, int a_col, const float* a2t, const float* a2_bias, const int* cu_tokens,
                          const int* state_slots, const int* fresh, float* state, float* out, float* prepared,
                          float q_scale, float tau, int tokens, int entries, int heads, int dim, int vdim, int rank,
                          cudaStream_t stream) {
    if (entries <= 0 || tokens <= 0) return 0;
    if (dim < 1 || vdim < 1 || rank < 1 || heads < 1 || !(tau > 0.0f)) return ME_ERR_ARGUMENT;
    if (static_cast<size_t>(PREP_TOKENS) * rank * sizeof(float) > 48 * 1024) return ME_ERR_UNSUPPORTED;
    PrepArgs p{proj, splits, static_cast<size_t>(split_stride), width, q_col, k_col, a_col, a2t, a2_bias, prepared,
               q_scale, 1.0f / tau, tokens, heads, dim, rank};
    // Few tokens: the channels of a token block are spread over several blocks as well.
    const int token_blocks = (tokens + PREP_TOKENS - 1) / PREP_TOKENS;
    const int channel_blocks = token_blocks >= 148 ? 1 : std::min((heads * dim + 255) / 256, 16);
    const int code = launch_kernel(gla_prepare_kernel, dim3(token_blocks, channel_blocks), 256,
                                   static_cast<size_t>(PREP_TOKENS) * rank * sizeof(float), stream, p);
    if (code) return code;
    ScanArgs a{proj, splits, static_cast<size_t>(split_stride), width, v_col, prepared, cu_tokens, state_slots,
               fresh, state, out, heads, dim, vdim};
    if (dim <= 16) return launch_scan<16>(a, entries, stream);
    if (dim <= 32) return launch_scan<32>(a, entries, stream);
    if (dim <= 64) return launch_scan<64>(a, entries, stream);
    if (dim <= 128) return launch_scan<128>(a, entries, stream);
    if (dim <= 192) return launch_scan<192>(a, entries, stream);
    return ME_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------- retention: a fixed decay per head

// Retention is the same recurrence with a constant decay per head in the place of the data-dependent one per
// channel, rotated queries and keys, and keys scaled by k_scale:
//
//   S_t = a_h S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t,  q_t = rot(W_q h_t),  k_t = rot(W_k h_t) * k_scale.
//
// Its prepare kernel fills the scan's input: the sums of the product's partial sums, the rotation of the first
// rotary_dim elements of every head (element e pairs with e + rotary_dim / 2, angles from the step's table), the
// key scale and the head's decay for every channel, float32.  The scan kernel above then walks the tokens.
struct RetentionPrepArgs {
    const float* proj;  // [splits][tokens][width]
    int splits;
    size_t split_stride;
    int width;
    int q_col, k_col;
    const float2* cos_sin;  // [tokens][rotary_dim / 2] or null
    const float* decay;     // [heads]
    float* prepared;        // [tokens][heads][3][dim]
    float k_scale;
    int tokens, heads, dim, rotary_dim;
};

__global__ void __launch_bounds__(256) retention_prepare_kernel(RetentionPrepArgs a) {
    const size_t total = static_cast<size_t>(a.tokens) * a.heads * a.dim;
    const int half = a.rotary_dim / 2;
    pdl_trigger();
    pdl_wait();
    for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int d = static_cast<int>(idx % a.dim);
        const int head = static_cast<int>((idx / a.dim) % a.heads);
        const size_t token = idx / (static_cast<size_t>(a.dim) * a.heads);
        const float* row = a.proj + token * a.width + head * a.dim;
        float q = 0.0f, k = 0.0f;
        for (int p = 0; p < a.splits; ++p) {
            q += row[p * a.split_stride + a.q_col + d];
            k += row[p * a.split_stride + a.k_col + d];
        }
        if (a.cos_sin && d < a.rotary_dim) {
            const int partner = d < half ? d + half : d - half;
            float q_other = 0.0f, k_other = 0.0f;
            for (int p = 0; p < a.splits; ++p) {
                q_other += row[p * a.split_stride + a.q_col + partner];
                k_other += row[p * a.split_stride + a.k_col + partner];
            }
            const float2 angle = a.cos_sin[token * half + (d < half ? d : d - half)];
            q = d < half ? q * angle.x - q_other * angle.y : q * angle.x + q_other * angle.y;
            k = d < half ? k * angle.x - k_other * angle.y : k * angle.x + k_other * angle.y;
        }
        float* dst = a.prepared + ((token * a.heads + head) * 3) * a.dim + d;
        dst[0] = q;
        dst[a.dim] = k * a.k_scale;
        dst[2 * a.dim] = a.decay[head];
    }
}

// ---------------------------------------------------- retention over long portions: chunks of 64 tokens

// With one decay per head the recurrence over a chunk of n tokens (S the state in front of it) has a closed form:
//
//   o_i   = a^(i + 1) S^T q_i + sum_(j <= i) a^(i - j) (q_i . k_j) v_j
//   S_new = a^n S + sum_j a^(n - 1 - j) k_j v_j^T
//
// so that a long portion runs as three kernels whose blocks work side by side instead of one warp walking the
// tokens: (1) every chunk's own sum of decayed k v^T; (2) per (request, head) the states in front of the chunks, one
// after the other, and the request's new state; (3) every chunk's outputs.  All of it is float32 on the CUDA cores
// with register tiles of 4 x 4 sums; a sum's order is fixed by the chunk's place in its portion, so a token's
// bits depend on how its request was cut into steps, by rounding only.  Entries with fewer than `min_count` tokens
// are left to the walking kernel above.
constexpr int RC = 64;
constexpr int STATE_ROWS = 32;   // rows of the state in front of a chunk that are staged at a time
constexpr int CHUNK_TILES = 4;   // 4 x 4 output tiles of a thread of the output kernel: vdim <= 256

struct ChunkArgs {
    const float* proj;  // [splits][tokens][width]: the value columns are read from here
    int splits;
    size_t split_stride;
    int width;
    int v_col;
    const float* prepared;  // [tokens][heads][3][dim]: rotated q, rotated and scaled k (the third part is not read)
    const float* decay;     // [heads]
    const int* cu_tokens;
    const int* state_slots;
    const int* fresh;
    float* state;        // [slots + 1][heads][dim][vdim]
    float* out;          // [tokens][heads][vdim]
    float* chunk_state;  // [chunks][heads][dim][vdim]: first every chunk's own sum, then the state in front of it
    int entries, heads, dim, vdim, min_count;
};

// The entry that chunk number `chunk` belongs to (entries of at least min_count tokens, cut in order).
__device__ __forceinline__ bool locate_chunk(const ChunkArgs& a, int chunk, int& entry, int& first_token, int& count) {
    int seen = 0;
    for (int b = 0; b < a.entries; ++b) {
        const int begin = a.cu_tokens[b], n = a.cu_tokens[b + 1] - begin;
        if (n < a.min_count) continue;
        const int chunks = (n + RC - 1) / RC;
        if (chunk < seen + chunks) {
            const int local = chunk - seen;
            entry = b, first_token = begin + local * RC, count = min(RC, n - local * RC);
            return true;
        }
        seen += chunks;
    }
    return false;
}

__device__ __forceinline__ float value_sum(const ChunkArgs& a, int token, int head, int e) {
    const float* src = a.proj + static_cast<size_t>(token) * a.width + a.v_col + head * a.vdim + e;
    float v = 0.0f;
    for (int p = 0; p < a.splits; ++p) v += src[p * a.split_stride];
    return v;
}

// (1) chunk_state[chunk][head] = sum_j a^(n - 1 - j) k_j v_j^T.  One block per (chunk, head).
__global__ void __launch_bounds__(256) retention_chunk_state_kernel(ChunkArgs a) {
    extern __shared__ __align__(16) float chunk_smem[];
    const int dim = a.dim, vdim = a.vdim, kd = dim + 4, vd = vdim + 4;
    float* kw = chunk_smem;           // [RC][dim + 4] keys times their decay up to the chunk's end
    float* v = kw + RC * kd;          // [RC][vdim + 4]
    __shared__ float pw[RC + 1];
    const int chunk = blockIdx.x, head = blockIdx.y;
    pdl_trigger();
    pdl_wait();
    int entry, first, count;
    if (!locate_chunk(a, chunk, entry, first, count)) return;
    const float decay = a.decay[head];
    for (int n = threadIdx.x; n <= RC; n += 256) pw[n] = powf(decay, static_cast<float>(n));
    __syncthreads();
    for (int i = threadIdx.x; i < count * dim; i += 256) {
        const int j = i / dim, d = i % dim;
        kw[j * kd + d] = a.prepared[((static_cast<size_t>(first + j) * a.heads + head) * 3 + 1) * dim + d] * pw[count - 1 - j];
    }
    for (int i = threadIdx.x; i < count * vdim; i += 256) {
        const int j = i / vdim, e = i % vdim;
        v[j * vd + e] = value_sum(a, first + j, head, e);
    }
    __syncthreads();
    const int across = vdim / 4, tiles = (dim / 4) * across;
    float* dst = a.chunk_state + (static_cast<size_t>(chunk) * a.heads + head) * dim * vdim;
    for (int t = threadIdx.x; t < tiles; t += 256) {
        const int dt = t / across, et = t % across;
        float acc[4][4] = {};
        for (int j = 0; j < count; ++j) {
            const float4 k4 = *reinterpret_cast<const float4*>(kw + j * kd + 4 * dt);
            const float4 v4 = *reinterpret_cast<const float4*>(v + j * vd + 4 * et);
            const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[r][c] = fmaf(kk[r], vv[c], acc[r][c]);
        }
#pragma unroll
        for (int r = 0; r < 4; ++r)
            *reinterpret_cast<float4*>(dst + static_cast<size_t>(4 * dt + r) * vdim + 4 * et) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
    }
}

// (2) Per (entry, head, four state elements): S walks the entry's chunks; chunk_state[c] becomes the state in front of
// chunk c, and the request's slot gets the state behind the last one.
__global__ void __launch_bounds__(256) retention_chunk_prefix_kernel(ChunkArgs a) {
    const int entry = blockIdx.x, head = blockIdx.y;
    const int quad = blockIdx.z * 256 + threadIdx.x;
    pdl_trigger();
    pdl_wait();
    const int per_head = a.dim * a.vdim;
    if (quad * 4 >= per_head) return;
    const int begin = a.cu_tokens[entry], n = a.cu_tokens[entry + 1] - begin;
    if (n < a.min_count) return;
    int first_chunk = 0;
    for (int b = 0; b < entry; ++b) {
        const int m = a.cu_tokens[b + 1] - a.cu_tokens[b];
        if (m >= a.min_count) first_chunk += (m + RC - 1) / RC;
    }
    const float decay = a.decay[head];
    float* slot = a.state + (static_cast<size_t>(a.state_slots[entry]) * a.heads + head) * per_head + quad * 4;
    float4 s = a.fresh[entry] ? make_float4(0.0f, 0.0f, 0.0f, 0.0f) : *reinterpret_cast<const float4*>(slot);
    const int chunks = (n + RC - 1) / RC;
    const float whole = powf(decay, static_cast<float>(RC));
    const size_t step = static_cast<size_t>(a.heads) * per_head;  // floats between two chunks of this head
    float* own = a.chunk_state + (static_cast<size_t>(first_chunk) * a.heads + head) * per_head + quad * 4;
    constexpr int AHEAD = 8;  // chunks whose sums are fetched together: the walk waits for memory once per AHEAD chunks
    for (int c0 = 0; c0 < chunks; c0 += AHEAD) {
        float4 sum[AHEAD];
#pragma unroll
        for (int i = 0; i < AHEAD; ++i)
            if (c0 + i < chunks) sum[i] = *reinterpret_cast<const float4*>(own + (c0 + i) * step);
#pragma unroll
        for (int i = 0; i < AHEAD; ++i) {
            const int c = c0 + i;
            if (c >= chunks) break;
            *reinterpret_cast<float4*>(own + c * step) = s;
            const int count = min(RC, n - c * RC);
            const float p = count == RC ? whole : powf(decay, static_cast<float>(count));
            s = make_float4(fmaf(p, s.x, sum[i].x), fmaf(p, s.y, sum[i].y), fmaf(p, s.z, sum[i].z), fmaf(p, s.w, sum[i].w));
        }
    }
    *reinterpret_cast<float4*>(slot) = s;
}

// (3) o_i = a^(i + 1) S^T q_i + sum_(j <= i) a^(i - j) (q_i . k_j) v_j with S = chunk_state[chunk][head].  One block per
// (chunk, head); thread (it, jt) owns rows it, it + 16, it + 32, it + 48 of a 4 x 4 tile, so that the 16-byte reads of
// eight neighbouring threads fall into different banks.
__global__ void __launch_bounds__(256, 2) retention_chunk_output_kernel(ChunkArgs a) {
    extern __shared__ __align__(16) float chunk_smem[];
    const int dim = a.dim, vdim = a.vdim, kd = dim + 4, vd = vdim + 4;
    constexpr int AD = RC + 1;
    float* q = chunk_smem;        // [RC][dim + 4]
    float* k = q + RC * kd;       // [RC][dim + 4] while the weights are formed; then the values take its place:
    float* v = k;                 // [RC][vdim + 4]
    float* w = k + RC * max(kd, vd);  // [RC][RC + 1]: a^(i - j) (q_i . k_j) for j <= i, else 0
    float* staged_state = w + RC * AD;  // [STATE_ROWS][vdim + 4]; every part before it holds a multiple of four floats
    __shared__ float pw[RC + 1];
    const int chunk = blockIdx.x, head = blockIdx.y;
    pdl_trigger();
    pdl_wait();
    int entry, first, count;
    if (!locate_chunk(a, chunk, entry, first, count)) return;
    const float decay = a.decay[head];
    for (int n = threadIdx.x; n <= RC; n += 256) pw[n] = powf(decay, static_cast<float>(n));
    for (int i = threadIdx.x; i < RC * dim; i += 256) {
        const int j = i / dim, d = i % dim;
        const float* src = a.prepared + ((static_cast<size_t>(first + j) * a.heads + head) * 3) * dim + d;
        q[j * kd + d] = j < count ? src[0] : 0.0f;
        k[j * kd + d] = j < count ? src[dim] : 0.0f;
    }
    __syncthreads();
    {
        const int it = threadIdx.x >> 4, jt = threadIdx.x & 15;
        float acc[4][4] = {};
        for (int d = 0; d < dim; d += 4) {
            float4 q4[4], k4[4];
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                q4[m] = *reinterpret_cast<const float4*>(q + (it + 16 * m) * kd + d);
                k4[m] = *reinterpret_cast<const float4*>(k + (jt + 16 * m) * kd + d);
            }
#pragma unroll
            for (int m = 0; m < 4; ++m)
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    acc[m][n] = fmaf(q4[m].x, k4[n].x, acc[m][n]);
                    acc[m][n] = fmaf(q4[m].y, k4[n].y, acc[m][n]);
                    acc[m][n] = fmaf(q4[m].z, k4[n].z, acc[m][n]);
                    acc[m][n] = fmaf(q4[m].w, k4[n].w, acc[m][n]);
                }
        }
#pragma unroll
        for (int m = 0; m < 4; ++m)
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                const int i = it + 16 * m, j = jt + 16 * n;
                w[i * AD + j] = j <= i ? acc[m][n] * pw[i - j] : 0.0f;
            }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < RC * vdim; i += 256) {  // the keys are done with: the values take their place
        const int j = i / vdim, e = i % vdim;
        v[j * vd + e] = j < count ? value_sum(a, first + j, head, e) : 0.0f;
    }
    // The state in front of the chunk comes through shared memory, STATE_ROWS rows at a time; a thread keeps the sums
    // of all its tiles (tiles t, t + 256, ...: at most CHUNK_TILES) over the passes.
    const int tiles = 16 * (vdim / 4);
    const float* front = a.chunk_state + (static_cast<size_t>(chunk) * a.heads + head) * dim * vdim;
    float acc[CHUNK_TILES][4][4] = {};
    for (int d0 = 0; d0 < dim; d0 += STATE_ROWS) {
        const int rows = min(STATE_ROWS, dim - d0), across = vdim / 4;
        for (int i = threadIdx.x; i < rows * across; i += 256) {
            const int r = i / across, c = i % across;
            *reinterpret_cast<float4*>(staged_state + r * vd + 4 * c) =
                __ldg(reinterpret_cast<const float4*>(front + static_cast<size_t>(d0 + r) * vdim + 4 * c));
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < CHUNK_TILES; ++u) {
            const int t = threadIdx.x + 256 * u;
            if (t >= tiles) continue;
            const int it = t & 15, et = t >> 4;
            for (int d = 0; d < rows; d += 4) {
                float4 q4[4], s4[4];
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    q4[m] = *reinterpret_cast<const float4*>(q + (it + 16 * m) * kd + d0 + d);
                    s4[m] = *reinterpret_cast<const float4*>(staged_state + (d + m) * vd + 4 * et);
                }
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    const float qq[4] = {q4[m].x, q4[m].y, q4[m].z, q4[m].w};
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        acc[u][m][0] = fmaf(qq[r], s4[r].x, acc[u][m][0]);
                        acc[u][m][1] = fmaf(qq[r], s4[r].y, acc[u][m][1]);
                        acc[u][m][2] = fmaf(qq[r], s4[r].z, acc[u][m][2]);
                        acc[u][m][3] = fmaf(qq[r], s4[r].w, acc[u][m][3]);
                    }
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int u = 0; u < CHUNK_TILES; ++u) {
        const int t = threadIdx.x + 256 * u;
        if (t >= tiles) continue;
        const int it = t & 15, et = t >> 4;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const float p = pw[it + 16 * m + 1];
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[u][m][c] *= p;
        }
        for (int j = 0; j < count; ++j) {  // the chunk's own tokens
            const float4 v4 = *reinterpret_cast<const float4*>(v + j * vd + 4 * et);
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                const float weight = w[(it + 16 * m) * AD + j];
                acc[u][m][0] = fmaf(weight, v4.x, acc[u][m][0]);
                acc[u][m][1] = fmaf(weight, v4.y, acc[u][m][1]);
                acc[u][m][2] = fmaf(weight, v4.z, acc[u][m][2]);
                acc[u][m][3] = fmaf(weight, v4.w, acc[u][m][3]);
            }
        }
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int i = it + 16 * m;
            if (i < count)
                *reinterpret_cast<float4*>(a.out + (static_cast<size_t>(first + i) * a.heads + head) * vdim + 4 * et) =
                    make_float4(acc[u][m][0], acc[u][m][1], acc[u][m][2], acc[u][m][3]);
        }
    }
}

static size_t chunk_output_smem(int dim, int vdim) {
    return (static_cast<size_t>(RC) * ((dim + 4) + std::max(dim + 4, vdim + 4)) + static_cast<size_t>(RC) * (RC + 1) +
            static_cast<size_t>(STATE_ROWS) * (vdim + 4)) * sizeof(float);
}

// Whether the chunked kernels take these head sizes (else every entry walks token by token).
ME_EXPORT int me_retention_chunked_supports(int dim, int vdim) {
    return dim >= 4 && vdim >= 4 && dim % 4 == 0 && vdim % 4 == 0 && vdim <= 64 * CHUNK_TILES &&
           chunk_output_smem(dim, vdim) <= 200 * 1024;
}

// `chunk_min`: entries of at least this many tokens run in chunks (0: none do), with `chunk_state` as scratch of
// `max_chunks * heads * dim * vdim` floats, max_chunks >= sum over those entries of ceil(tokens / 64).
ME_EXPORT int me_retention_scan(const float* proj, int splits, long long split_stride, int width, int q_col, int k_col,
                                int v_col, const float* cos_sin, int rotary_dim, const float* decay, float k_scale,
                                const int* cu_tokens, const int* state_slots, const int* fresh, float* state, float* out,
                                float* prepared, int tokens, int entries, int heads, int dim, int vdim, int chunk_min,
                                float* chunk_state, int max_chunks, cudaStream_t stream) {
    if (entries <= 0 || tokens <= 0) return 0;
    if (dim < 1 || vdim < 1 || heads < 1 || rotary_dim < 0 || rotary_dim > dim || rotary_dim % 2) return ME_ERR_ARGUMENT;
    RetentionPrepArgs p{proj, splits, static_cast<size_t>(split_stride), width, q_col, k_col,
                        reinterpret_cast<const float2*>(cos_sin), decay, prepared, k_scale, tokens, heads, dim, rotary_dim};
    const size_t total = static_cast<size_t>(tokens) * heads * dim;
    const int blocks = static_cast<int>(std::min<size_t>((total + 255) / 256, 148 * 16));
    int code = launch_kernel(retention_prepare_kernel, blocks, 256, 0, stream, p);
    if (code) return code;
    if (chunk_min > 0) {
        if (!me_retention_chunked_supports(dim, vdim) || chunk_state == nullptr || max_chunks < 1) return ME_ERR_ARGUMENT;
        ChunkArgs c{proj, splits, static_cast<size_t>(split_stride), width, v_col, prepared, decay, cu_tokens, state_slots,
                    fresh, state, out, chunk_state, entries, heads, dim, vdim, chunk_min};
        static SharedMemoryOptIn state_opt_in, output_opt_in;
        const size_t state_smem = static_cast<size_t>(RC) * ((dim + 4) + (vdim + 4)) * sizeof(float);
        const size_t output_smem = chunk_output_smem(dim, vdim);
        // The opt-in is remembered per device, so it is made for the largest size that is ever accepted.
        if ((code = state_opt_in(retention_chunk_state_kernel, 200 * 1024))) return code;
        if ((code = output_opt_in(retention_chunk_output_kernel, 200 * 1024))) return code;
        if ((code = launch_kernel_in_order(retention_chunk_state_kernel, dim3(max_chunks, heads), 256, state_smem, stream, c))) return code;
        const dim3 prefix_grid(entries, heads, (dim * vdim / 4 + 255) / 256);
        if ((code = launch_kernel_in_order(retention_chunk_prefix_kernel, prefix_grid, 256, 0, stream, c))) return code;
        if ((code = launch_kernel_in_order(retention_chunk_output_kernel, dim3(max_chunks, heads), 256, output_smem, stream, c))) return code;
    }
    ScanArgs a{proj, splits, static_cast<size_t>(split_stride), width, v_col, prepared, cu_tokens, state_slots,
               fresh, state, out, heads, dim, vdim, chunk_min > 0 ? chunk_min - 1 : 0};
    if (dim <= 16) return launch_scan<16>(a, entries, stream);
    if (dim <= 32) return launch_scan<32>(a, entries, stream);
    if (dim <= 64) return launch_scan<64>(a, entries, stream);
    if (dim <= 128) return launch_scan<128>(a, entries, stream);
    if (dim <= 192) return launch_scan<192>(a, entries, stream);
    return ME_ERR_UNSUPPORTED;
}

// out[t][h][e] = weight[e] * o[t][h][e] * rsqrt(mean_e(o^2) + eps) * silu(gate[t][h][e]); a null weight is all ones.
template <typename T>
__global__ void __launch_bounds__(128) gla_finish_kernel(const float* __restrict__ o, const float* __restrict__ proj,
                                                         int splits, size_t split_stride, int width, int g_col,
                                                         const float* __restrict__ weight, float eps,
                                                         T* __restrict__ out, int tokens, int heads, int vdim) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = static_cast<long long>(blockIdx.x) * 4 + warp;
    pdl_trigger();
    pdl_wait();
    if (item >= static_cast<long long>(tokens) * heads) return;
    const size_t token = static_cast<size_t>(item / heads);
    const int head = static_cast<int>(item % heads);
    const float* row = o + (token * heads + head) * vdim;
    float sum_sq = 0.0f;
    for (int e = lane; e < vdim; e += 32) sum_sq = fmaf(row[e], row[e], sum_sq);
    sum_sq = warp_sum(sum_sq);
    const float inv = rsqrtf(sum_sq / static_cast<float>(vdim) + eps);
    const float* gate_row = proj + token * width + g_col + head * vdim;
    T* dst = out + (token * heads + head) * vdim;
    for (int e = lane; e < vdim; e += 32) {
        float gate = 0.0f;
        for (int p = 0; p < splits; ++p) gate += gate_row[p * split_stride + e];
        const float activated = gate / (1.0f + expf(-gate));
        dst[e] = from_float<T>((weight ? weight[e] : 1.0f) * (row[e] * inv) * activated);
    }
}

ME_EXPORT int me_gla_finish(const float* o, const float* proj, int splits, long long split_stride, int width,
                            int g_col, const float* weight, float eps, void* out, int type, int tokens, int heads,
                            int vdim, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const long long items = static_cast<long long>(tokens) * heads;
    const int blocks = static_cast<int>((items + 3) / 4);
    if (type == ME_BF16)
        return launch_kernel(gla_finish_kernel<__nv_bfloat16>, blocks, 128, 0, stream, o, proj, splits,
                             (size_t)split_stride, width, g_col, weight, eps, static_cast<__nv_bfloat16*>(out), tokens,
                             heads, vdim);
    return launch_kernel(gla_finish_kernel<float>, blocks, 128, 0, stream, o, proj, splits, (size_t)split_stride, width,
                         g_col, weight, eps, static_cast<float*>(out), tokens, heads, vdim);
}
