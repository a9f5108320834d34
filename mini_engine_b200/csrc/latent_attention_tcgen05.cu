// Attention of prompt portions over a cache of latent rows with both products on tcgen05.
//
// The cache holds one row [c | k_rot] of `width` elements per token that is key for every head and, in its first
// `R` elements, value (latent_attention.cu has the algebra).  The rows of a score tile are (token, head) pairs, 128
// consecutive ones of a request to a CTA; all of them meet the same keys, in tiles of 64 keys that start at
// multiples of 64 in absolute position.  The output of 128 rows x R columns of 32-bit sums is as large as the whole
// tensor memory, so two CTAs share a row block: each forms all scores and probabilities of the block and the half
// of the output columns that blockIdx.x names (the scores are computed twice; the second product, the larger one
// per key for R = 512, is not).
//
//   warp 0    fetches the 128 query rows once and every key tile by TMA, page by page, in 64-column blocks
//             (128-byte swizzle); pages behind the window or past the last key are never named
//   warp 1    owns tensor memory and issues the MMAs: S[128 x 64] = Q K^T over width / 16 steps, then
//             O[128 x R/2] += P C with P read from tensor memory and C being this CTA's columns of the key tile
//   warps 2-5 one thread per row: scale, mask (causal edge and window), running maximum with the output rescaled
//             only when some row's maximum has grown by more than 2^8, probabilities rounded to bfloat16 over the
//             scores' own columns, row sums in float32; at the end O / sum * gate -> out
//
// Query rows take 128 x width x 2 bytes of shared memory and a key tile 64 x width x 2, so for widths up to 576 one
// key tile fits beside the queries: of the next tile, the columns that this CTA's second product does not read are
// fetched as soon as the scores are done, the others when the second product has read this tile.  Every wait
// is bounded (tcgen05.cuh); a wait that ran out sets an error code, and the CTA frees its tensor memory and returns.
#include "tcgen05.cuh"

constexpr int LT_ROWS = 128;
constexpr int LT_KEYS = 64;
constexpr int LT_THREADS = 192;
constexpr int LT_TMEM_COLUMNS = 512;
constexpr int LT_Q_BLOCK = LT_ROWS * 128;  // bytes of a 64-column block of the query tile
constexpr int LT_K_BLOCK = LT_KEYS * 128;  // and of the key tile
constexpr float LT_LOG2E = 1.4426950408889634f;

__device__ int g_latent_tc_error = 0;

struct LatentTcParams {
    const int* block_table;   // [entries][table_width]
    const int* cu_tokens;     // [entries + 1]
    const int* context_lens;  // [entries]
    const int* entry_ids;     // the batch entries this launch covers (grid.z of them), or null: all
    __nv_bfloat16* out;       // [tokens][heads][R]
    const float* gate;        // [tokens][heads] or null
    float scale_log2;
    int heads, width, rank, page_size, table_width, window;
};

__device__ __forceinline__ float lt_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float lt_max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ uint32_t lt_pack(float lo, float hi) {
    uint32_t packed;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(hi), "f"(lo));
    return packed;
}

// grid (2 column halves, row blocks, entries)
__global__ void __launch_bounds__(LT_THREADS, 1)
latent_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                LatentTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int blocks = p.width / 64;  // 64-column blocks of a row
    uint8_t* q_tile = tiles;                       // [blocks][128 rows][64]
    uint8_t* k_tile = tiles + blocks * LT_Q_BLOCK;  // [blocks][64 keys][64]
    uint64_t* bars = reinterpret_cast<uint64_t*>(k_tile + blocks * LT_K_BLOCK);
    // The key tile has two parts with barriers of their own: the 64-column blocks that this CTA's second product
    // reads as values ("c": free when that product is done) and the others ("rest": free when the scores are done, so
    // that the next tile's share of them arrives while this tile's softmax and second product run).
    uint64_t *q_full = bars, *c_full = bars + 1, *c_empty = bars + 2, *s_full = bars + 3, *p_full = bars + 4,
             *o_full = bars + 5, *rest_full = bars + 7, *rest_empty = bars + 8;  // o_full: two, by the tile's parity
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 9);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = blockIdx.x;
    const int row_block = gridDim.y - 1 - blockIdx.y;  // later blocks see more keys: they start first
    const int half_columns = p.rank / 2;
    const int c_blocks = half_columns / 64, c_first = half * c_blocks;  // the blocks [c_first, c_first + c_blocks) are values here

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(c_full, 1);
        mbar_init(c_empty, 1);
        mbar_init(rest_full, 1);
        mbar_init(rest_empty, 1);
        mbar_init(s_full, 1);
        mbar_init(p_full, LT_ROWS);
        mbar_init(o_full, 1);
        mbar_init(o_full + 1, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tcgen05_alloc(tmem_holder, LT_TMEM_COLUMNS);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_s = *tmem_holder;  // S, then P over its first 32 columns
    const uint32_t tmem_o = tmem_s + LT_KEYS;

    pdl_trigger();
    pdl_wait();
    const int entry = p.entry_ids ? p.entry_ids[blockIdx.z] : blockIdx.z;
    const int token0 = p.cu_tokens[entry];
    const int new_tokens = p.cu_tokens[entry + 1] - token0;
    const int rows_total = new_tokens * p.heads;
    const int row0 = row_block * LT_ROWS;
    const bool has_work = row0 < rows_total;  // uniform for the CTA
    const int rows_valid = min(LT_ROWS, rows_total - row0);
    const int context = p.context_lens[entry];
    const int first_pos = context - new_tokens;
    const int pos_lo = first_pos + row0 / p.heads, pos_hi = first_pos + (row0 + rows_valid - 1) / p.heads;
    const int lowest = p.window > 0 ? max(pos_lo - p.window + 1, 0) : 0;  // the first key that the first row sees
    const int first_tile = lowest / LT_KEYS;
    const int tiles_count = has_work ? pos_hi / LT_KEYS + 1 - first_tile : 0;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (has_work) {
            const int* table = p.block_table + static_cast<size_t>(entry) * p.table_width;
            const int pages_per_tile = LT_KEYS / p.page_size;
            const int first_page_index = lowest / p.page_size, last_page_index = (context - 1) / p.page_size;
            const int page_bytes = p.page_size * 128;  // one page of one 64-column block
            if (lane == 0) {
                mbar_expect_tx(q_full, blocks * LT_Q_BLOCK);
                for (int b = 0; b < blocks; ++b)
                    tma_load_2d(q_tile + b * LT_Q_BLOCK, &map_q, b * 64, token0 * p.heads + row0, q_full);
            }
            const bool loads = lane < pages_per_tile;
            bool ok = true;
            for (int j = 0; j < tiles_count && ok; ++j) {
                // Page indices are held inside [the page of the first visible key, the page of the last key]: a page
                // behind the window may have been given back, and what a row must not see is masked anyway.
                const int index = min(max((first_tile + j) * pages_per_tile + lane, first_page_index), last_page_index);
                const int page = loads ? table[index] : 0;
                for (int part = 0; part < 2 && ok; ++part) {  // the rest first: it comes free first
                    uint64_t* empty = part ? c_empty : rest_empty;
                    uint64_t* full = part ? c_full : rest_full;
                    if (lane == 0) {
                        ok = mbar_wait(empty, (j & 1) ^ 1);
                        if (ok) mbar_expect_tx(full, (part ? c_blocks : blocks - c_blocks) * LT_K_BLOCK);
                        else atomicCAS(&g_latent_tc_error, 0, (1 << 8) | part);
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (ok && loads)
                        for (int b = 0; b < blocks; ++b)
                            if ((b >= c_first && b < c_first + c_blocks) == (part == 1))
                                tma_load_2d(k_tile + b * LT_K_BLOCK + lane * page_bytes, &map_k, b * 64, page * p.page_size, full);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && has_work) {
            constexpr uint32_t idesc_s = make_idesc(LT_KEYS);  // S[128 x 64] = Q K^T, K-major operands
            const uint32_t idesc_o = make_idesc(half_columns, true);  // O[128 x R/2] += P C, C is MN-major
            const uint32_t c_tile = smem_u32(k_tile) + c_first * LT_K_BLOCK;  // this CTA's columns
            bool ok = mbar_wait(q_full, 0);
            if (!ok) atomicCAS(&g_latent_tc_error, 0, 2 << 8);
            for (int j = 0; j < tiles_count && ok; ++j) {
                const uint32_t parity = j & 1;
                ok = mbar_wait(rest_full, parity) && mbar_wait(c_full, parity);
                if (!ok) { atomicCAS(&g_latent_tc_error, 0, (2 << 8) | 1); break; }
                tcgen05_fence_after();
                // The S columns are free once the previous second product has read P out of them: the MMAs of a
                // CTA execute in the order of their issue.
                for (int kk = 0; kk < p.width / 16; ++kk) {
                    const uint32_t q_offset = (kk / 4) * LT_Q_BLOCK + (kk % 4) * 32, k_offset = (kk / 4) * LT_K_BLOCK + (kk % 4) * 32;
                    tcgen05_mma_bf16(tmem_s, smem_desc_sw128(smem_u32(q_tile) + q_offset),
                                     smem_desc_sw128(smem_u32(k_tile) + k_offset), idesc_s, kk > 0 ? 1u : 0u);
                }
                tcgen05_commit(s_full);
                tcgen05_commit(rest_empty);
                ok = mbar_wait(p_full, parity);
                if (!ok) { atomicCAS(&g_latent_tc_error, 0, (2 << 8) | 2); break; }
                tcgen05_fence_after();
#pragma unroll
                for (int kk = 0; kk < LT_KEYS / 16; ++kk) {
                    // 16 keys = 16 rows of 128 bytes; the next 64 columns are one block further
                    const uint64_t c_desc = smem_desc_sw128_mn(c_tile + kk * 16 * 128, LT_K_BLOCK);
                    tcgen05_mma_bf16_ts(tmem_o, tmem_s + kk * 8, c_desc, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
                }
                tcgen05_commit(o_full + (j & 1));
                tcgen05_commit(c_empty);
            }
        }
    } else if (has_work) {
        // ------------------------------------------------------------------ softmax rows
        const int quarter = warp & 3;  // this warp's tensor-memory lanes are [32 * quarter, +32)
        const int row = quarter * 32 + lane;
        const int row_pos = first_pos + (row0 + min(row, rows_valid - 1)) / p.heads;
        const int lowest_seen = p.window > 0 ? row_pos - p.window + 1 : 0;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        float row_max = -INFINITY, row_sum = 0.0f;
        bool ok = true;
        int j = 0;
        for (; j < tiles_count && ok; ++j) {
            const uint32_t parity = j & 1;
            ok = mbar_wait(s_full, parity);
            if (!ok) break;
            tcgen05_fence_after();
            const int first_key = (first_tile + j) * LT_KEYS;
            // Only the tiles at the causal edge and at the window's edge hold keys that some row must not see.
            const bool masked_tile = first_key + LT_KEYS - 1 > pos_lo || (p.window > 0 && first_key < pos_hi - p.window + 1);
            uint32_t raw[64];
            tcgen05_ld32_nowait(tmem_s + lane_base, raw);
            tcgen05_ld32_nowait(tmem_s + lane_base + 32, raw + 32);
            tcgen05_wait_ld();
            tcgen05_pin32(raw);
            tcgen05_pin32(raw + 32);
            // raw stays unscaled (the scale is positive, so the maximum may be taken first); masked scores are -inf
            float best[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (masked_tile) {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    if (first_key + i > row_pos || first_key + i < lowest_seen) raw[i] = __float_as_uint(-INFINITY);
                    best[i & 3] = fmaxf(best[i & 3], __uint_as_float(raw[i]));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 64; i += 2)  // two scores per instruction
                    best[(i >> 1) & 3] = lt_max3(best[(i >> 1) & 3], __uint_as_float(raw[i]), __uint_as_float(raw[i + 1]));
            }
            const float tile_max = fmaxf(fmaxf(best[0], best[1]), fmaxf(best[2], best[3])) * p.scale_log2;
            // The row's reference value follows its true maximum lazily: O is rescaled (and the second product of
            // the tile before waited for) only when the maximum of some row of the warp has grown by more than 2^8;
            // until then probabilities are taken relative to the older reference and may exceed 1.
            const float new_max = fmaxf(row_max, tile_max);
            if (j == 0) {
                row_max = new_max;
            } else if (__any_sync(0xffffffffu, new_max - row_max > 8.0f)) {
                ok = mbar_wait(o_full + ((j - 1) & 1), ((j - 1) >> 1) & 1);  // the MMAs run in order: all of O is complete
                if (!ok) break;
                tcgen05_fence_after();
                // a row that has seen no key yet: its sum and output are zero and stay so
                const float rescale = row_max == -INFINITY ? 1.0f : exp2f(row_max - new_max);
                row_sum *= rescale;
                row_max = new_max;
#pragma unroll 1
                for (int c = 0; c < half_columns / 16; ++c) {
                    float o[16];
                    tcgen05_ld16(tmem_o + lane_base + c * 16, o);
                    uint32_t scaled[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) scaled[i] = __float_as_uint(o[i] * rescale);
                    tcgen05_st16(tmem_o + lane_base + c * 16, scaled);
                }
            }
            const float base = row_max == -INFINITY ? 0.0f : row_max;
            // exp2(score * scale - base) for two scores at a time with the two-wide float32 instructions
            const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), base2 = make_float2(-base, -base);
            float2 partial[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float2 x = __ffma2_rn(make_float2(__uint_as_float(raw[c * 32 + i]), __uint_as_float(raw[c * 32 + i + 1])), scale2, base2);
                    const float2 pr = make_float2(lt_exp2(x.x), lt_exp2(x.y));  // 2^-inf = 0
                    partial[(i >> 1) & 1] = __fadd2_rn(partial[(i >> 1) & 1], pr);
                    packed[i / 2] = lt_pack(pr.x, pr.y);
                }
                tcgen05_st16(tmem_s + lane_base + c * 16, packed);  // P columns [16 c, +16) hold keys [32 c, +32)
            }
            row_sum += (partial[0].x + partial[0].y) + (partial[1].x + partial[1].y);
            tcgen05_wait_st();
            tcgen05_fence_before();
            mbar_arrive(p_full);
        }
        if (ok && j == tiles_count) ok = mbar_wait(o_full + ((tiles_count - 1) & 1), ((tiles_count - 1) >> 1) & 1);
        if (!ok) atomicCAS(&g_latent_tc_error, 0, 3 << 8);
        if (ok) {
            tcgen05_fence_after();
            const size_t pair_index = static_cast<size_t>(token0) * p.heads + row0 + row;  // token * heads + head
            const bool valid = row < rows_valid;
            const float whole = valid ? (p.gate ? p.gate[pair_index] : 1.0f) / row_sum : 0.0f;
            __nv_bfloat16* dst = p.out + pair_index * p.rank + half * half_columns;
#pragma unroll 1
            for (int c = 0; c < half_columns / 32; ++c) {
                float o[32];
                tcgen05_ld32(tmem_o + lane_base + c * 32, o);  // collective: every lane takes part
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 chunk;
                        chunk.x = lt_pack(o[i] * whole, o[i + 1] * whole);
                        chunk.y = lt_pack(o[i + 2] * whole, o[i + 3] * whole);
                        chunk.z = lt_pack(o[i + 4] * whole, o[i + 5] * whole);
                        chunk.w = lt_pack(o[i + 6] * whole, o[i + 7] * whole);
                        *reinterpret_cast<uint4*>(dst + c * 32 + i) = chunk;
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) tcgen05_dealloc(tmem_s, LT_TMEM_COLUMNS);
}

// -------------------------------------------------------------------------------- host

ME_EXPORT int me_latent_attention_tcgen05_take_error(int* code) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(code, g_latent_tc_error, sizeof(int));
    if (e != cudaSuccess) return static_cast<int>(e);
    if (*code != 0) e = cudaMemcpyToSymbol(g_latent_tc_error, &zero, sizeof(int));
    return static_cast<int>(e);
}

// Dynamic shared memory of a CTA: the query and key tiles, room to align them to 1,024 bytes, barriers.
static size_t latent_tc_smem(int width) { return static_cast<size_t>(width / 64) * (LT_Q_BLOCK + LT_K_BLOCK) + 1024 + 256; }

// q is described by a TMA map (me_make_tensor_map, gemm_tcgen05.cu) as [tokens * heads][width] with boxes of 128
// rows x 64 columns, the pages as [(pages * page_size)][width] with boxes of page_size rows.  `longest`: the most new
// tokens that an entry of the launch brings.
ME_EXPORT int me_latent_attention_tcgen05(const void* map_q, const void* map_k, const int* block_table, const int* cu_tokens,
                                          const int* context_lens, void* out, const float* gate, const int* entry_ids,
                                          float scale, int entries, int longest, int heads, int width, int rank,
                                          int page_size, int table_width, int window, cudaStream_t stream) {
    if (entries <= 0 || longest <= 0) return 0;
    if (heads < 1 || window < 0) return ME_ERR_ARGUMENT;
    if (width % 64 || rank % 128 || rank < 128 || rank > 512 || rank > width) return ME_ERR_UNSUPPORTED;
    if (page_size < 8 || page_size > LT_KEYS || LT_KEYS % page_size) return ME_ERR_UNSUPPORTED;
    const size_t smem = latent_tc_smem(width);
    if (smem > 227 * 1024) return ME_ERR_UNSUPPORTED;
    alignas(64) CUtensorMap q, k;
    memcpy(&q, map_q, sizeof(q));
    memcpy(&k, map_k, sizeof(k));
    LatentTcParams p{block_table, cu_tokens, context_lens, entry_ids, static_cast<__nv_bfloat16*>(out), gate,
                     scale * LT_LOG2E, heads, width, rank, page_size, table_width, window};
    const long long rows = static_cast<long long>(longest) * heads;
    static SharedMemoryOptIn opt_in;
    if (const int e = opt_in(latent_attention_tcgen05_kernel, 227 * 1024)) return e;  // once per device: the most any width needs
    return launch_kernel(latent_attention_tcgen05_kernel, dim3(2, static_cast<unsigned>((rows + LT_ROWS - 1) / LT_ROWS), entries),
                         LT_THREADS, smem, stream, q, k, p);
}
