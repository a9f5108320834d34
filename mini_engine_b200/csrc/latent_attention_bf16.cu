// Attention over a cache of latent rows in bfloat16 with tensor-core products, and the per-head products around it.
//
// The cache holds one row [c | k_rot] of `width` elements per token; every head's query has already been mapped
// into that space, so all heads share the one row as key, and the first `R` elements of the same row are the value
// (see latent_attention.cu for the algebra).  All heads of a token see the same keys, so the rows of a score tile
// are (token, head) pairs: a CTA takes 32 consecutive pairs of one request (two tokens of 16 heads, a quarter of a
// token's 128 heads) and walks the keys they can see in tiles of 64 that start at multiples of 64 in absolute
// position, double-buffered through shared memory.  Eight warps, two steps per tile:
//
//   scores   warp (row half, key quarter): 16 rows x 16 keys over the whole width, A and B by ldmatrix;
//            mask, scale, running maximum (exchanged between the four warps of a row half through shared memory),
//            probabilities rounded to bfloat16 into a shared tile;
//   values   warp (row half, value quarter): acc[16 x R/4] += P[16 x 64] C[64 x R/4], C being the key tile itself.
//
// Scores, maxima, sums and the output accumulate in float32.  Keys outside the visible range are zero-filled in
// shared memory and never read from the cache.  Requests that bring one token split their keys over several CTAs
// (spans of 128 keys by absolute position, so the split depends on the position only); each writes a partial
// (maximum, sum, unnormalised output) and a second launch of one CTA per (token, head) merges them in ascending key order.
//
// head_product_bf16: out[t][h][n] = sum_k x[t][h][k] W[h][k][n] on the same instructions: a CTA takes 64 tokens of
// one head and 128 outputs, x rounded to bfloat16 once (it may arrive as float32 partial sums), W streamed in slabs of
// 64 k.  `tail` more columns per head are rotated and appended, as in the plain kernel.
#include "mma_sync.cuh"

constexpr int LAT_ROWS = 32;      // (token, head) pairs per CTA
constexpr int LAT_KEYS = 64;      // keys per tile
constexpr int LAT_THREADS = 256;  // eight warps
constexpr int LAT_SPAN = 128;     // keys of one CTA of a split request
constexpr float LAT_LOG2E = 1.4426950408889634f;
constexpr int LAT_MAX_SMEM = 226 * 1024;  // dynamic shared memory a CTA may ask for (the kernel has a few static bytes too)

struct LatentParams {
    const __nv_bfloat16* q;      // [tokens][heads][width]
    const __nv_bfloat16* pages;  // [pages][page_size][width]
    const int* block_table;      // [entries][table_width]
    const int* cu_tokens;        // [entries + 1]
    const int* context_lens;     // [entries]
    __nv_bfloat16* out;          // [tokens][heads][R]
    const float* gate;           // [tokens][heads] multiplier of each head's output, or null
    float* partials;             // split: [entries][heads][max_splits][R + 2]
    const int* entry_ids;        // the batch entries this launch covers (grid.z of them), or null: all, in order
    float scale_log2;            // scale * log2(e)
    int heads, width, page_size, table_width, window, max_splits;
};

__device__ int g_latent_error = 0;  // 2: a request needed more partial-result slots than the launch was given

__device__ __forceinline__ long long latent_row_offset(const LatentParams& p, const int* table, int key, int lowest, int last_key) {
    if (key < lowest || key > last_key) return -1;
    const int page_index = key / p.page_size;
    const int page = table[page_index];
    if (page < 0) return -1;
    return (static_cast<long long>(page) * p.page_size + (key - page_index * p.page_size)) * p.width;
}

// grid (row blocks, splits, entries).  SPLIT: every entry of the launch brings one token.
template <int R, bool SPLIT>
__global__ void __launch_bounds__(LAT_THREADS, 1) latent_attention_kernel(LatentParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int chunks = p.width / 8;  // 16-byte chunks of a row
    __nv_bfloat16* q_tile = reinterpret_cast<__nv_bfloat16*>(smem);                   // [32][width]
    __nv_bfloat16* k_tiles = q_tile + LAT_ROWS * p.width;                              // [2 stages][64][width]
    __nv_bfloat16* p_tile = k_tiles + 2 * LAT_KEYS * p.width;                          // [32][64]
    float* tile_max = reinterpret_cast<float*>(p_tile + LAT_ROWS * LAT_KEYS);          // [4 key quarters][32]
    float* sums = tile_max + 4 * LAT_ROWS;                                             // [4 key quarters][32]
    constexpr int NV = R / 32;  // 8-wide value tiles of one warp (a quarter of R)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = warp & 1, quarter = warp >> 1;
    pdl_trigger();
    pdl_wait();
    const int entry = p.entry_ids ? p.entry_ids[blockIdx.z] : blockIdx.z;
    const int token0 = p.cu_tokens[entry];
    const int new_tokens = p.cu_tokens[entry + 1] - token0;
    const int rows_total = new_tokens * p.heads;
    // Later blocks of a request see more keys: start them first so that the grid's tail is short.
    const int row_block = SPLIT ? blockIdx.x : gridDim.x - 1 - blockIdx.x;
    const int row0 = row_block * LAT_ROWS;
    if (row0 >= rows_total) return;
    const int rows_valid = min(LAT_ROWS, rows_total - row0);
    const int first_pos = p.context_lens[entry] - new_tokens;  // position of the entry's first new token
    const int pos_lo = first_pos + row0 / p.heads, pos_hi = first_pos + (row0 + rows_valid - 1) / p.heads;
    int lowest = p.window > 0 ? max(pos_lo - p.window + 1, 0) : 0;
    int last_key = pos_hi;
    int slot = 0, first_slot = 0, last_slot = 0;
    if (SPLIT) {
        first_slot = lowest / LAT_SPAN, last_slot = pos_hi / LAT_SPAN;
        if (last_slot - first_slot >= p.max_splits) {
            atomicCAS(&g_latent_error, 0, 2);
            last_slot = first_slot + p.max_splits - 1;
        }
        slot = first_slot + blockIdx.y;
        if (slot > last_slot) return;
        lowest = max(lowest, slot * LAT_SPAN);
        last_key = min(last_key, slot * LAT_SPAN + LAT_SPAN - 1);
    }
    const int* table = p.block_table + static_cast<size_t>(entry) * p.table_width;

    // Queries of this block -> shared memory (rows past the end are zero).  An entry's rows are contiguous.
    {
        const __nv_bfloat16* q_src = p.q + (static_cast<size_t>(token0) * p.heads + row0) * p.width;
        for (int idx = threadIdx.x; idx < LAT_ROWS * chunks; idx += LAT_THREADS) {
            const int row = idx / chunks, chunk = idx - row * chunks;
            const bool valid = row < rows_valid;
            cp_async_16(q_tile + swizzled_at(row, chunk, chunks) * 8,
                        valid ? q_src + static_cast<size_t>(row) * p.width + chunk * 8 : p.q, valid);
        }
    }
    const int first_tile = lowest / LAT_KEYS, last_tile = last_key / LAT_KEYS;
    auto prefetch = [&](int tile, int stage) {
        __nv_bfloat16* k_tile = k_tiles + stage * LAT_KEYS * p.width;
        // a warp fetches whole rows: lane 0's page lookup serves the row
        for (int row = warp; row < LAT_KEYS; row += LAT_THREADS / 32) {
            const long long offset = latent_row_offset(p, table, tile * LAT_KEYS + row, lowest, last_key);
            const bool valid = offset >= 0;
            for (int chunk = lane; chunk < chunks; chunk += 32)
                cp_async_16(k_tile + swizzled_at(row, chunk, chunks) * 8, p.pages + (valid ? offset + chunk * 8 : 0), valid);
        }
    };
    prefetch(first_tile, 0);
    cp_async_commit();

    float acc[NV][4];
#pragma unroll
    for (int n = 0; n < NV; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
    int row_pos[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = min(half * 16 + (lane >> 2) + r * 8, rows_valid - 1);
        row_pos[r] = first_pos + (row0 + row) / p.heads;
    }

    for (int tile = first_tile; tile <= last_tile; ++tile) {
        const int stage = (tile - first_tile) & 1;
        if (tile < last_tile) {
            prefetch(tile + 1, stage ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const __nv_bfloat16* k_tile = k_tiles + stage * LAT_KEYS * p.width;

        // scores of 16 rows x 16 keys
        float s[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[n][i] = 0.0f;
        {
            const int a_row = half * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            const int b_key = quarter * 16 + (lane & 7) + (lane >> 4) * 8;
            const int steps = p.width / 16;
#pragma unroll 4
            for (int kk = 0; kk < steps; ++kk) {
                uint32_t a[4], b[4];
                ldmatrix_x4(a, q_tile + swizzled_at(a_row, kk * 2 + (lane >> 4), chunks) * 8);
                ldmatrix_x4(b, k_tile + swizzled_at(b_key, kk * 2 + ((lane >> 3) & 1), chunks) * 8);
                mma_bf16(s[0], a, b[0], b[1]);
                mma_bf16(s[1], a, b[2], b[3]);
            }
        }
        // mask, scale, this warp's maximum per row
        const int col0 = tile * LAT_KEYS + quarter * 16 + 2 * (lane & 3);
        float mine[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int key = col0 + n * 8 + (i & 1), r = i >> 1;
                const bool visible = key <= row_pos[r] && key >= lowest && key <= last_key &&
                                     (p.window <= 0 || key > row_pos[r] - p.window);
                s[n][i] = visible ? s[n][i] * p.scale_log2 : -INFINITY;
                mine[r] = fmaxf(mine[r], s[n][i]);
            }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mine[r] = fmaxf(mine[r], __shfl_xor_sync(0xffffffffu, mine[r], 1));
            mine[r] = fmaxf(mine[r], __shfl_xor_sync(0xffffffffu, mine[r], 2));
            if ((lane & 3) == 0) tile_max[quarter * LAT_ROWS + half * 16 + (lane >> 2) + r * 8] = mine[r];
        }
        __syncthreads();
        float rescale[2], base[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = half * 16 + (lane >> 2) + r * 8;
            float new_max = row_max[r];
#pragma unroll
            for (int w = 0; w < 4; ++w) new_max = fmaxf(new_max, tile_max[w * LAT_ROWS + row]);
            base[r] = new_max == -INFINITY ? 0.0f : new_max;  // a row that has seen nothing yet
            rescale[r] = exp2f(row_max[r] - base[r]);         // 0 while row_max is -inf
            row_max[r] = new_max;
            row_sum[r] *= rescale[r];
        }
        // probabilities -> the shared tile, rounded once; this warp's part of the row sums
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const float p0 = exp2f(s[n][r * 2] - base[r]), p1 = exp2f(s[n][r * 2 + 1] - base[r]);
                row_sum[r] += p0 + p1;
                const int row = half * 16 + (lane >> 2) + r * 8;
                const int col = quarter * 16 + n * 8 + 2 * (lane & 3);
                *reinterpret_cast<uint32_t*>(p_tile + swizzled<LAT_KEYS>(row, col >> 3) * 8 + (col & 7)) = pack_bf16(p0, p1);
            }
#pragma unroll
        for (int n = 0; n < NV; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[n][i] *= rescale[i >> 1];
        __syncthreads();
        // acc[16 x R/4] += P[16 x 64] C[64 x R/4]
#pragma unroll
        for (int kk = 0; kk < LAT_KEYS / 16; ++kk) {
            uint32_t a[4];
            const int a_row = half * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            ldmatrix_x4(a, p_tile + swizzled<LAT_KEYS>(a_row, kk * 2 + (lane >> 4)) * 8);
            const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
            for (int pair = 0; pair < NV / 2; ++pair) {
                uint32_t b[4];
                const int chunk = quarter * NV + pair * 2 + (lane >> 4);
                ldmatrix_x4_trans(b, k_tile + swizzled_at(key, chunk, chunks) * 8);
                mma_bf16(acc[pair * 2], a, b[0], b[1]);
                mma_bf16(acc[pair * 2 + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();  // the next iteration's prefetch and probabilities overwrite what was read here
    }

    // The rows' sums: four lanes of a warp, then the four warps of a row half, in a fixed order.
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
        if ((lane & 3) == 0) sums[quarter * LAT_ROWS + half * 16 + (lane >> 2) + r * 8] = row_sum[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = half * 16 + (lane >> 2) + r * 8;
        row_sum[r] = (sums[row] + sums[LAT_ROWS + row]) + (sums[2 * LAT_ROWS + row] + sums[3 * LAT_ROWS + row]);
    }

    if (!SPLIT) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = half * 16 + (lane >> 2) + r * 8;
            if (row >= rows_valid) continue;
            const size_t pair_index = static_cast<size_t>(token0) * p.heads + row0 + row;  // token * heads + head
            const float whole = (p.gate ? p.gate[pair_index] : 1.0f) / row_sum[r];
            __nv_bfloat16* dst = p.out + pair_index * R + quarter * (R / 4);
#pragma unroll
            for (int n = 0; n < NV; ++n)
                *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * (lane & 3)) = pack_bf16(acc[n][r * 2] * whole, acc[n][r * 2 + 1] * whole);
        }
        return;
    }

    // A split request: this CTA's partial (unnormalised output, maximum, sum) of every row it holds.
    constexpr int STRIDE = R + 2;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = half * 16 + (lane >> 2) + r * 8;
        if (row >= rows_valid) continue;
        float* dst = p.partials + ((static_cast<size_t>(entry) * p.heads + row0 + row) * p.max_splits + blockIdx.y) * STRIDE;
#pragma unroll
        for (int n = 0; n < NV; ++n)
            *reinterpret_cast<float2*>(dst + quarter * (R / 4) + n * 8 + 2 * (lane & 3)) = make_float2(acc[n][r * 2], acc[n][r * 2 + 1]);
        if (quarter == 0 && (lane & 3) == 0) dst[R] = row_max[r], dst[R + 1] = row_sum[r];
    }
}

// The partials of a split request -> out: grid (heads, entries), one (token, head) row per CTA.  The weight of a
// partial is exp2(its maximum - the maximum of all), zero for one that saw no key; weighted sums and outputs are added
// in ascending order of the keys, so the result depends on the positions alone.
template <int R>
__global__ void __launch_bounds__(128) latent_merge_kernel(LatentParams p) {
    extern __shared__ float merge_smem[];  // weights [max_splits], weight * sum [max_splits]
    __shared__ float warp_max[4];
    __shared__ float total_shared;
    constexpr int STRIDE = R + 2;
    const int head = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    const int entry = p.entry_ids ? p.entry_ids[blockIdx.y] : blockIdx.y;
    const int pos = p.context_lens[entry] - 1;  // the entry's one new token
    const int lowest = p.window > 0 ? max(pos - p.window + 1, 0) : 0;
    const int active = min(pos / LAT_SPAN - lowest / LAT_SPAN + 1, p.max_splits);
    const size_t pair_index = static_cast<size_t>(p.cu_tokens[entry]) * p.heads + head;
    const float* part = p.partials + (static_cast<size_t>(entry) * p.heads + head) * p.max_splits * STRIDE;
    float* weights = merge_smem;
    float* weighted = merge_smem + p.max_splits;
    float total_max = -INFINITY;
    for (int sl = threadIdx.x; sl < active; sl += 128) total_max = fmaxf(total_max, part[sl * STRIDE + R]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) total_max = fmaxf(total_max, __shfl_xor_sync(0xffffffffu, total_max, d));
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = total_max;
    __syncthreads();
    total_max = fmaxf(fmaxf(warp_max[0], warp_max[1]), fmaxf(warp_max[2], warp_max[3]));
    for (int sl = threadIdx.x; sl < active; sl += 128) {
        const float m = part[sl * STRIDE + R];
        const float weight = m == -INFINITY ? 0.0f : exp2f(m - total_max);
        weights[sl] = weight;
        weighted[sl] = part[sl * STRIDE + R + 1] * weight;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int sl = 0; sl < active; ++sl) total += weighted[sl];
        total_shared = total;
    }
    __syncthreads();
    const float whole = (p.gate ? p.gate[pair_index] : 1.0f) / total_shared;
    for (int col = threadIdx.x * 2; col < R; col += 256) {
        float2 value = make_float2(0.0f, 0.0f);
        int sl = 0;
        for (; sl + 4 <= active; sl += 4) {
            float2 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = *reinterpret_cast<const float2*>(part + (sl + j) * STRIDE + col);
#pragma unroll
            for (int j = 0; j < 4; ++j) value.x = fmaf(v[j].x, weights[sl + j], value.x), value.y = fmaf(v[j].y, weights[sl + j], value.y);
        }
        for (; sl < active; ++sl) {
            const float2 v = *reinterpret_cast<const float2*>(part + sl * STRIDE + col);
            value.x = fmaf(v.x, weights[sl], value.x), value.y = fmaf(v.y, weights[sl], value.y);
        }
        *reinterpret_cast<uint32_t*>(p.out + pair_index * R + col) = pack_bf16(value.x * whole, value.y * whole);
    }
}

ME_EXPORT int me_latent_attention_bf16_take_error(int* code) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(code, g_latent_error, sizeof(int));
    if (e != cudaSuccess) return static_cast<int>(e);
    if (*code != 0) e = cudaMemcpyToSymbol(g_latent_error, &zero, sizeof(int));
    return static_cast<int>(e);
}

static SharedMemoryOptIn g_latent_opt_in[8];

template <int R, bool SPLIT>
static int launch_latent(const LatentParams& p, dim3 grid, size_t smem, cudaStream_t stream, int slot) {
    auto kernel = latent_attention_kernel<R, SPLIT>;
    int code = g_latent_opt_in[slot](kernel, LAT_MAX_SMEM);  // once per device: the most any width needs
    if (code != 0) return code;
    code = launch_kernel(kernel, grid, LAT_THREADS, smem, stream, p);
    if (code != 0 || !SPLIT) return code;
    const size_t merge_smem = 2 * static_cast<size_t>(p.max_splits) * sizeof(float);
    if (merge_smem > 40 * 1024) return ME_ERR_UNSUPPORTED;
    return launch_kernel(latent_merge_kernel<R>, dim3(p.heads, grid.z), 128, merge_smem, stream, p);
}

// `longest`: the most new tokens that an entry of the launch brings; `split` != 0: every entry brings one token,
// `max_splits` CTAs share the keys of a (request, row block), `partials` is given, and a second launch merges them
// (`counters` is not used).
ME_EXPORT int me_latent_attention_bf16(const void* q, const void* pages, const int* block_table, const int* cu_tokens,
                                       const int* context_lens, void* out, const float* gate, float* partials,
                                       int* counters, const int* entry_ids, float scale, int entries, int longest,
                                       int heads, int width, int rank, int page_size, int table_width, int window,
                                       int split, int max_splits, cudaStream_t stream) {
    if (entries <= 0 || longest <= 0) return 0;
    if (width % 64 || width < 64 || rank > width || heads < 1) return ME_ERR_UNSUPPORTED;
    if (split && (partials == nullptr || max_splits < 1 || longest != 1)) return ME_ERR_ARGUMENT;
    LatentParams p{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(pages), block_table, cu_tokens,
                   context_lens, static_cast<__nv_bfloat16*>(out), gate, partials, entry_ids,
                   scale * LAT_LOG2E, heads, width, page_size, table_width, window, max_splits};
    const size_t smem = (static_cast<size_t>(LAT_ROWS + 2 * LAT_KEYS) * width + LAT_ROWS * LAT_KEYS) * sizeof(__nv_bfloat16) +
                        8 * LAT_ROWS * sizeof(float);
    if (smem > LAT_MAX_SMEM) return ME_ERR_UNSUPPORTED;
    const long long rows = static_cast<long long>(longest) * heads;
    const dim3 grid(static_cast<unsigned>((rows + LAT_ROWS - 1) / LAT_ROWS), split ? max_splits : 1, entries);
    switch (rank) {
        case 128: return split ? launch_latent<128, true>(p, grid, smem, stream, 0) : launch_latent<128, false>(p, grid, smem, stream, 1);
        case 256: return split ? launch_latent<256, true>(p, grid, smem, stream, 2) : launch_latent<256, false>(p, grid, smem, stream, 3);
        case 384: return split ? launch_latent<384, true>(p, grid, smem, stream, 4) : launch_latent<384, false>(p, grid, smem, stream, 5);
        case 512: return split ? launch_latent<512, true>(p, grid, smem, stream, 6) : launch_latent<512, false>(p, grid, smem, stream, 7);
    }
    return ME_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------------ products per head

constexpr int HPT_TOKENS = 64;   // tokens per CTA (16 per warp)
constexpr int HPT_OUTS = 128;    // outputs per CTA
constexpr int HPT_SLAB = 64;     // k per slab of the weights
constexpr int HPT_THREADS = 128;

struct HeadProductParams {
    const void* in;  // [splits][tokens][heads * (inner + tail)] float partial sums, or [tokens][...] bfloat16
    int splits;
    size_t split_stride;
    const __nv_bfloat16* weight;  // [heads][inner][outs]
    const float2* cos_sin;        // [tokens][rotary_dim / 2] or null
    __nv_bfloat16* out;           // [tokens][heads][outs + tail]
    int tokens, heads, inner, outs, tail, rotary_dim;
    int chunks_per_cta;  // consecutive output chunks of 128 that one CTA walks with the same x tile
};

// grid (token tiles, heads, groups of output chunks of 128).
template <bool FLOAT_IN>
__global__ void __launch_bounds__(HPT_THREADS) head_product_bf16_kernel(HeadProductParams a) {
    extern __shared__ __align__(128) uint8_t smem[];
    __nv_bfloat16* x_tile = reinterpret_cast<__nv_bfloat16*>(smem);  // [64][inner]
    __nv_bfloat16* w_slabs = x_tile + HPT_TOKENS * a.inner;          // [2 stages][64 k][128 outputs]
    const int head = blockIdx.y, first = blockIdx.x * HPT_TOKENS;
    const int chunk0 = blockIdx.z * a.chunks_per_cta;
    const int my_chunks = min(a.chunks_per_cta, (a.outs + HPT_OUTS - 1) / HPT_OUTS - chunk0);
    const int slabs = a.inner / HPT_SLAB;
    const int count = min(HPT_TOKENS, a.tokens - first);
    const int in_head = a.inner + a.tail, out_head = a.outs + a.tail;
    const int chunks = a.inner / 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const __nv_bfloat16* weight = a.weight + static_cast<size_t>(head) * a.inner * a.outs;
    auto fetch_slab = [&](int item, int stage) {  // item: (output chunk, slab) in the order they are used
        const int n0 = (chunk0 + item / slabs) * HPT_OUTS, slab = item % slabs;
        __nv_bfloat16* dst = w_slabs + stage * HPT_SLAB * HPT_OUTS;
        for (int idx = threadIdx.x; idx < HPT_SLAB * (HPT_OUTS / 8); idx += HPT_THREADS) {
            const int k = idx / (HPT_OUTS / 8), chunk = idx % (HPT_OUTS / 8);
            const bool valid = n0 + chunk * 8 < a.outs;
            cp_async_16(dst + swizzled<HPT_OUTS>(k, chunk) * 8,
                        valid ? weight + static_cast<size_t>(slab * HPT_SLAB + k) * a.outs + n0 + chunk * 8 : a.weight, valid);
        }
    };
    pdl_trigger();
    fetch_slab(0, 0);  // weights: no kernel writes them
    cp_async_commit();
    pdl_wait();
    // x of this head -> shared memory as bfloat16 (rows past the end are zero)
    int x_done = 0;
    if (FLOAT_IN && a.splits == 1) {  // whole sums: four chunks of eight per thread with all their loads in flight
        for (; x_done + 4 * HPT_THREADS <= HPT_TOKENS * chunks; x_done += 4 * HPT_THREADS) {
            float4 lo[4], hi[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = x_done + u * HPT_THREADS + threadIdx.x;
                const int t = idx / chunks, chunk = idx - t * chunks;
                lo[u] = hi[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (t < count) {
                    const float* src = static_cast<const float*>(a.in) + (static_cast<size_t>(first + t) * a.heads + head) * in_head + chunk * 8;
                    lo[u] = *reinterpret_cast<const float4*>(src), hi[u] = *reinterpret_cast<const float4*>(src + 4);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = x_done + u * HPT_THREADS + threadIdx.x;
                const int t = idx / chunks, chunk = idx - t * chunks;
                *reinterpret_cast<uint4*>(x_tile + swizzled_at(t, chunk, chunks) * 8) =
                    make_uint4(pack_bf16(lo[u].x, lo[u].y), pack_bf16(lo[u].z, lo[u].w), pack_bf16(hi[u].x, hi[u].y), pack_bf16(hi[u].z, hi[u].w));
            }
        }
    }
    for (int idx = x_done + threadIdx.x; idx < HPT_TOKENS * chunks; idx += HPT_THREADS) {
        const int t = idx / chunks, chunk = idx - t * chunks;
        __nv_bfloat16* dst = x_tile + swizzled_at(t, chunk, chunks) * 8;
        const size_t at = (static_cast<size_t>(first + t) * a.heads + head) * in_head + chunk * 8;
        if (FLOAT_IN) {
            float v[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
            if (t < count) {
                const float* src = static_cast<const float*>(a.in) + at;
                for (int s = 0; s < a.splits; ++s) {
                    const float4 lo = *reinterpret_cast<const float4*>(src + s * a.split_stride);
                    const float4 hi = *reinterpret_cast<const float4*>(src + s * a.split_stride + 4);
                    v[0] += lo.x, v[1] += lo.y, v[2] += lo.z, v[3] += lo.w, v[4] += hi.x, v[5] += hi.y, v[6] += hi.z, v[7] += hi.w;
                }
            }
            *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
        } else {
            const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(a.in);
            cp_async_16(dst, t < count ? src + at : src, t < count);
        }
    }
    cp_async_commit();  // x is a group of its own: the first wait of the loop below covers it
    float acc[HPT_OUTS / 8][4];
#pragma unroll
    for (int n = 0; n < HPT_OUTS / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;
    const int items = my_chunks * slabs;
    for (int item = 0; item < items; ++item) {
        const int stage = item & 1, slab = item % slabs;
        if (item + 1 < items) {
            fetch_slab(item + 1, stage ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const __nv_bfloat16* w_slab = w_slabs + stage * HPT_SLAB * HPT_OUTS;
#pragma unroll
        for (int kk = 0; kk < HPT_SLAB / 16; ++kk) {
            uint32_t x[4];
            const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            ldmatrix_x4(x, x_tile + swizzled_at(row, (slab * (HPT_SLAB / 16) + kk) * 2 + (lane >> 4), chunks) * 8);
            const int k = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
            for (int pair = 0; pair < HPT_OUTS / 16; ++pair) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, w_slab + swizzled<HPT_OUTS>(k, pair * 2 + (lane >> 4)) * 8);
                mma_bf16(acc[pair * 2], x, b[0], b[1]);
                mma_bf16(acc[pair * 2 + 1], x, b[2], b[3]);
            }
        }
        __syncthreads();  // the next iteration's slab overwrites the other stage's reader
        if (slab != slabs - 1) continue;
        // the chunk is whole: out it goes, and the sums start again
        const int n0 = (chunk0 + item / slabs) * HPT_OUTS;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int t = warp * 16 + (lane >> 2) + r * 8;
            __nv_bfloat16* dst = a.out + (static_cast<size_t>(first + t) * a.heads + head) * out_head + n0;
#pragma unroll
            for (int n = 0; n < HPT_OUTS / 8; ++n) {
                const int col = n * 8 + 2 * (lane & 3);
                if (t < count && n0 + col < a.outs) *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(acc[n][r * 2], acc[n][r * 2 + 1]);
                acc[n][r * 2] = acc[n][r * 2 + 1] = 0.0f;
            }
        }
    }
    if (blockIdx.z != 0 || a.tail == 0) return;
    // the tail: the rotated part of every head, from the 32-bit sums
    const int half = a.rotary_dim / 2;
    for (int i = threadIdx.x; i < count * a.tail; i += HPT_THREADS) {
        const int t = i / a.tail, e = i % a.tail;
        const size_t at = (static_cast<size_t>(first + t) * a.heads + head) * in_head + a.inner;
        auto element = [&](int j) {
            if (!FLOAT_IN) return __bfloat162float(static_cast<const __nv_bfloat16*>(a.in)[at + j]);
            float v = 0.0f;
            for (int s = 0; s < a.splits; ++s) v += static_cast<const float*>(a.in)[s * a.split_stride + at + j];
            return v;
        };
        float value = element(e);
        if (a.cos_sin && e < a.rotary_dim) {
            const float other = element(e < half ? e + half : e - half);
            const float2 angle = a.cos_sin[static_cast<size_t>(first + t) * half + (e < half ? e : e - half)];
            value = e < half ? value * angle.x - other * angle.y : value * angle.x + other * angle.y;
        }
        a.out[(static_cast<size_t>(first + t) * a.heads + head) * out_head + a.outs + e] = __float2bfloat16_rn(value);
    }
}

static SharedMemoryOptIn g_head_product_opt_in[2];

// in_type: ME_F32 for float input (partial sums allowed), ME_BF16 for bfloat16 input (one split).
ME_EXPORT int me_head_product_bf16(const void* in, int in_type, int splits, long long split_stride, const void* weight,
                                   const float* cos_sin, void* out, int tokens, int heads, int inner, int outs, int tail,
                                   int rotary_dim, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (heads < 1 || tail < 0 || rotary_dim < 0 || rotary_dim > tail || rotary_dim % 2) return ME_ERR_ARGUMENT;
    if (in_type != ME_F32 && splits != 1) return ME_ERR_ARGUMENT;
    if (inner % 64 || inner < 64 || outs % 8 || outs < 8 || tail % 8) return ME_ERR_UNSUPPORTED;
    const size_t smem = (static_cast<size_t>(HPT_TOKENS) * inner + 2 * HPT_SLAB * HPT_OUTS) * sizeof(__nv_bfloat16);
    if (smem > 200 * 1024) return ME_ERR_UNSUPPORTED;
    HeadProductParams a{in, splits, static_cast<size_t>(split_stride), static_cast<const __nv_bfloat16*>(weight),
                        reinterpret_cast<const float2*>(cos_sin), static_cast<__nv_bfloat16*>(out),
                        tokens, heads, inner, outs, tail, rotary_dim, 1};
    // Many token tiles: one CTA walks all output chunks of its (tile, head), so x is fetched and rounded once.
    // Few: a CTA per chunk, for the parallelism.
    const int out_chunks = (outs + HPT_OUTS - 1) / HPT_OUTS;
    if (static_cast<long long>((tokens + HPT_TOKENS - 1) / HPT_TOKENS) * heads >= 2 * 148) a.chunks_per_cta = out_chunks;
    const dim3 grid((tokens + HPT_TOKENS - 1) / HPT_TOKENS, heads, (out_chunks + a.chunks_per_cta - 1) / a.chunks_per_cta);
    if (in_type == ME_F32) {
        auto kernel = head_product_bf16_kernel<true>;
        const int code = g_head_product_opt_in[0](kernel, 200 * 1024);  // once per device: the most any size needs
        return code != 0 ? code : launch_kernel(kernel, grid, HPT_THREADS, smem, stream, a);
    }
    auto kernel = head_product_bf16_kernel<false>;
    const int code = g_head_product_opt_in[1](kernel, 200 * 1024);
    return code != 0 ? code : launch_kernel(kernel, grid, HPT_THREADS, smem, stream, a);
}
