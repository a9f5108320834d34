// The router of a feed-forward made of many small units ("experts") of which a token uses a few.
//
// Per token: z = W_r h (+ a bias per unit) in float32 (h in the compute dtype, W_r float32), s = sigmoid(z); in
// mode 1, s = z itself and the chosen units' weights are the softmax over the chosen logits only.  The units form
// `group_count` equal groups of neighbours; a group's value is the sum of its two largest scores (of its
// only score when a group is a single unit) and only units of the `group_keep` best groups are eligible.
// Among those the `top` largest scores are chosen; their weights are s / (sum of the chosen s + 1e-20) *
// weight_scale.  Ties go to the lower index.  The kernel leaves a dense map `weights [T][units]` (zero for
// units that were not chosen), and the chosen units and their weights as lists `[T][top]`.
//
// One block per token: warp w forms the scores of units w, w + 8, ...; one thread then chooses.  The sums
// run over the columns in a fixed order, so a token's choice never depends on the rest of the batch.
#include "common.cuh"

constexpr int ROUTE_WARPS = 8;
constexpr int MAX_UNITS = 1024;

struct RouteArgs {
    const void* h;        // [tokens][hidden]
    const float* router;  // [units][hidden]
    const float* bias;    // [units] added to the logits, or null
    int mode;             // 0: sigmoid scores over their sum; 1: the largest logits, softmax over the chosen ones
    float* weights;       // [tokens][units]
    int* chosen;          // [tokens][top]
    float* chosen_weight; // [tokens][top]
    int tokens, hidden, units, top, group_count, group_keep;
    float weight_scale;
};

template <typename T>
__global__ void __launch_bounds__(ROUTE_WARPS * 32) route_kernel(RouteArgs a) {
    __shared__ float score[MAX_UNITS];
    __shared__ unsigned char eligible[MAX_UNITS];
    const int token = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_trigger();
    pdl_wait();
    const T* h = static_cast<const T*>(a.h) + static_cast<size_t>(token) * a.hidden;
    // Lane l adds the products of columns 4 l .. 4 l + 3 (+ 128 j) in ascending order into four sums of its own, which
    // are then added in a fixed order: many loads in flight, and a token's scores are the same bits in every step.
    const bool quads = a.hidden % 4 == 0 && reinterpret_cast<uintptr_t>(a.router) % 16 == 0 && reinterpret_cast<uintptr_t>(a.h) % 8 == 0;
    for (int unit = warp; unit < a.units; unit += ROUTE_WARPS) {
        const float* w = a.router + static_cast<size_t>(unit) * a.hidden;
        float sum = 0.0f;
        if (quads) {
            float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
            for (int i = lane * 4; i < a.hidden; i += 128) {
                const float4 weight = *reinterpret_cast<const float4*>(w + i);
                part[0] = fmaf(to_float(h[i]), weight.x, part[0]);
                part[1] = fmaf(to_float(h[i + 1]), weight.y, part[1]);
                part[2] = fmaf(to_float(h[i + 2]), weight.z, part[2]);
                part[3] = fmaf(to_float(h[i + 3]), weight.w, part[3]);
            }
            sum = (part[0] + part[1]) + (part[2] + part[3]);
        } else {
            for (int i = lane; i < a.hidden; i += 32) sum = fmaf(to_float(h[i]), w[i], sum);
        }
        sum = warp_sum(sum);
        if (a.bias) sum += a.bias[unit];
        if (lane == 0) score[unit] = a.mode == 1 ? sum : 1.0f / (1.0f + expf(-sum));
    }
    for (int unit = threadIdx.x; unit < a.units; unit += ROUTE_WARPS * 32) {
        eligible[unit] = 0;
        a.weights[static_cast<size_t>(token) * a.units + unit] = 0.0f;
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    const int per = a.units / a.group_count;
    // The best groups, one at a time (group counts are small).
    for (int turn = 0; turn < a.group_keep; ++turn) {
        int best = -1;
        float best_value = -INFINITY;
        for (int g = 0; g < a.group_count; ++g) {
            if (eligible[g * per]) continue;  // taken in an earlier turn
            float first = -INFINITY, second = -INFINITY;
            for (int u = g * per; u < (g + 1) * per; ++u) {
                const float s = score[u];
                if (s > first) second = first, first = s;
                else if (s > second) second = s;
            }
            const float value = per > 1 ? first + second : first;
            if (value > best_value) best_value = value, best = g;
        }
        if (best < 0) break;
        for (int u = best * per; u < (best + 1) * per; ++u) eligible[u] = 1;
    }
    float total = 0.0f;
    int* chosen = a.chosen + static_cast<size_t>(token) * a.top;
    float* chosen_weight = a.chosen_weight + static_cast<size_t>(token) * a.top;
    for (int turn = 0; turn < a.top; ++turn) {
        int best = -1;
        float best_score = -INFINITY;
        for (int u = 0; u < a.units; ++u)
            if (eligible[u] == 1 && score[u] > best_score) best_score = score[u], best = u;
        chosen[turn] = best;
        if (best < 0) continue;
        eligible[best] = 2;
        total += best_score;
    }
    float inv = a.weight_scale / (total + 1e-20f), top_logit = 0.0f;
    if (a.mode == 1) {  // exp(z - max) over the sum of the chosen: the first choice holds the largest logit
        top_logit = chosen[0] >= 0 ? score[chosen[0]] : 0.0f;
        float denom = 0.0f;
        for (int turn = 0; turn < a.top; ++turn)
            if (chosen[turn] >= 0) denom += expf(score[chosen[turn]] - top_logit);
        inv = a.weight_scale / denom;
    }
    for (int turn = 0; turn < a.top; ++turn) {
        const int u = chosen[turn];
        const float weight = u < 0 ? 0.0f : a.mode == 1 ? expf(score[u] - top_logit) * inv : score[u] * inv;
        chosen_weight[turn] = weight;
        if (u >= 0) a.weights[static_cast<size_t>(token) * a.units + u] = weight;
    }
}

ME_EXPORT int me_route(const void* h, int h_type, const float* router, const float* bias, int mode, float* weights,
                       int* chosen, float* chosen_weight, int tokens, int hidden, int units, int top, int group_count,
                       int group_keep, float weight_scale, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (units < 1 || units > MAX_UNITS) return ME_ERR_UNSUPPORTED;
    if (group_count < 1 || units % group_count || group_keep < 1 || group_keep > group_count || top < 1 ||
        top > group_keep * (units / group_count))
        return ME_ERR_ARGUMENT;
    if (mode != 0 && mode != 1) return ME_ERR_ARGUMENT;
    RouteArgs a{h, router, bias, mode, weights, chosen, chosen_weight, tokens, hidden, units, top, group_count, group_keep, weight_scale};
    if (h_type == ME_BF16) return launch_kernel(route_kernel<__nv_bfloat16>, tokens, ROUTE_WARPS * 32, 0, stream, a);
    return launch_kernel(route_kernel<float>, tokens, ROUTE_WARPS * 32, 0, stream, a);
}

// ------------------------------------------------------------- rows sorted by unit, for grouped products

// From the lists `chosen [T][top]`: every (token, choice) gets a row in an array that is sorted by unit, each unit's
// run padded to a multiple of `pad` rows.  Leaves `row_of [T * top]` (the row of each choice), `token_of [capacity]`
// (the token of each row, -1 for padding and for the unused tail) and `unit_of_block [capacity / pad]` (the unit of
// every run of `pad` rows, -1 where no rows are).  One CTA; the order of a unit's rows among themselves is not
// fixed, and nothing depends on it: a row's products do not depend on its place.
constexpr int SORT_THREADS = 1024;

__global__ void __launch_bounds__(SORT_THREADS) sort_by_unit_kernel(const int* __restrict__ chosen, int items, int units, int pad,
                                                                    int capacity, int* __restrict__ row_of,
                                                                    int* __restrict__ token_of, int* __restrict__ unit_of_block,
                                                                    int top) {
    __shared__ int count[MAX_UNITS], first[MAX_UNITS];
    pdl_trigger();
    pdl_wait();
    for (int u = threadIdx.x; u < units; u += SORT_THREADS) count[u] = 0;
    for (int r = threadIdx.x; r < capacity; r += SORT_THREADS) token_of[r] = -1;
    for (int b = threadIdx.x; b < capacity / pad; b += SORT_THREADS) unit_of_block[b] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < items; i += SORT_THREADS) {
        const int u = chosen[i];
        if (u >= 0) atomicAdd(&count[u], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int row = 0;
        for (int u = 0; u < units; ++u) {
            first[u] = row;
            const int blocks = (count[u] + pad - 1) / pad;
            for (int b = 0; b < blocks; ++b) unit_of_block[row / pad + b] = u;
            row += blocks * pad;
            count[u] = 0;  // becomes the cursor of the unit's run
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < items; i += SORT_THREADS) {
        const int u = chosen[i];
        if (u < 0) { row_of[i] = -1; continue; }
        const int row = first[u] + atomicAdd(&count[u], 1);
        row_of[i] = row;
        token_of[row] = i / top;
    }
}

// sorted[row] = h[token_of[row]] (zeros for rows without a token), 16 bytes per thread and step.
__global__ void gather_rows_kernel(const uint4* __restrict__ h, const int* __restrict__ token_of, uint4* __restrict__ sorted,
                                   int rows, int chunks) {
    pdl_trigger();
    pdl_wait();
    const size_t total = static_cast<size_t>(rows) * chunks;
    for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int row = static_cast<int>(idx / chunks), chunk = static_cast<int>(idx % chunks);
        const int token = token_of[row];
        sorted[idx] = token >= 0 ? h[static_cast<size_t>(token) * chunks + chunk] : make_uint4(0u, 0u, 0u, 0u);
    }
}

// out[t] = sum over the token's choices, in their order, of weight[t][k] * sorted_out[row_of[t][k]], float32.
__global__ void combine_rows_kernel(const float* __restrict__ sorted_out, const int* __restrict__ row_of,
                                    const float* __restrict__ weight, float* __restrict__ out, int tokens, int top, int width) {
    pdl_trigger();
    pdl_wait();
    const size_t total = static_cast<size_t>(tokens) * width;
    for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int t = static_cast<int>(idx / width), c = static_cast<int>(idx % width);
        float sum = 0.0f;
        for (int k = 0; k < top; ++k) {
            const int row = row_of[t * top + k];
            if (row >= 0) sum = fmaf(weight[t * top + k], sorted_out[static_cast<size_t>(row) * width + c], sum);
        }
        out[idx] = sum;
    }
}

ME_EXPORT int me_sort_by_unit(const int* chosen, int tokens, int top, int units, int pad, int capacity, int* row_of,
                              int* token_of, int* unit_of_block, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (units < 1 || units > MAX_UNITS || pad < 1 || capacity % pad) return ME_ERR_ARGUMENT;
    // every unit's run may end in a partly filled block
    if (static_cast<long long>(capacity) < static_cast<long long>(tokens) * top + static_cast<long long>(units) * (pad - 1))
        return ME_ERR_ARGUMENT;
    return launch_kernel(sort_by_unit_kernel, 1, SORT_THREADS, 0, stream, chosen, tokens * top, units, pad, capacity, row_of,
                         token_of, unit_of_block, top);
}

ME_EXPORT int me_gather_rows(const void* h, const int* token_of, void* sorted, int rows, int row_bytes, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (row_bytes % 16 || reinterpret_cast<uintptr_t>(h) % 16 || reinterpret_cast<uintptr_t>(sorted) % 16) return ME_ERR_ARGUMENT;
    const int chunks = row_bytes / 16;
    const size_t total = static_cast<size_t>(rows) * chunks;
    const int blocks = static_cast<int>((total + 255) / 256 < 148 * 32 ? (total + 255) / 256 : 148 * 32);
    return launch_kernel(gather_rows_kernel, blocks, 256, 0, stream, static_cast<const uint4*>(h), token_of,
                         static_cast<uint4*>(sorted), rows, chunks);
}

ME_EXPORT int me_combine_rows(const float* sorted_out, const int* row_of, const float* weight, float* out, int tokens, int top,
                              int width, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const size_t total = static_cast<size_t>(tokens) * width;
    const int blocks = static_cast<int>((total + 255) / 256 < 148 * 32 ? (total + 255) / 256 : 148 * 32);
    return launch_kernel(combine_rows_kernel, blocks, 256, 0, stream, sorted_out, row_of, weight, out, tokens, top, width);
}
