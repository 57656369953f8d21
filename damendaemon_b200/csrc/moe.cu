// Experts chosen per token by a table: the bookkeeping around the grouped products.
//
// A token uses K of E experts. The (token, choice) pairs are laid out expert by expert in a buffer of rows in
// which every expert's rows start on a multiple of the product's row tile, so that a tile of rows meets one
// expert's matrices only (tile_group[tile] = that expert, or -1 for a tile no pair fell into):
//
//   dd_route_by_table   token ids + table [vocab, K] -> pair_row [N*K] (the row of pair (t, k)), row_token [rows]
//                       (the token of a row, -1 for a row of padding), tile_group [rows / tile]
//   dd_gather_rows      x [N, width] -> sorted rows (a row of padding is zeroed)
//                       (ids null: token t reads row t of the table, which then holds the step's own choices)
//   dd_route_by_score   normed rows [N, width] and the router's matrix -> float32 logits, then the K experts of every token
//                       by score within the worthiest groups, their weights, and the gate of a shared unit
//   dd_gated_unit       rows of [gate | up] halves -> y = f(gate, up) in float32 (dd_gated_value in common.cuh: the
//                       clamped form g * sigmoid(alpha g) * (u + 1), silu(gate) * up, or tanh-gelu(gate) * up),
//                       optionally times a number per row
//   dd_combine_rows     stream[t] += sum over k of weight (* pair_weight[t*K + k]) * y[pair_row[t*K + k]], k ascending,
//                       in float32
//
// The order of an expert's rows among themselves depends on the order in which threads arrive; no value depends
// on it, since every row is computed by itself and the sum over a token's experts runs in the order of its choices.
#include "common.cuh"

namespace {
constexpr int ROUTE_THREADS = 1024;

__global__ void __launch_bounds__(ROUTE_THREADS)
route_by_table_kernel(const int* __restrict__ ids, const int* __restrict__ table, int n_tokens, int vocab, int top,
                      int n_experts, int tile, int n_rows, int* __restrict__ pair_row, int* __restrict__ row_token,
                      int* __restrict__ tile_group, int* __restrict__ error_flag) {
    extern __shared__ int shared[];              // [E] counts, then cursors; [E + 1] first rows
    int* count = shared;
    int* first = shared + n_experts;
    dd_launch_dependents();
    dd_grid_wait();
    const int n_pairs = n_tokens * top;
    for (int e = threadIdx.x; e < n_experts; e += ROUTE_THREADS) count[e] = 0;
    for (int r = threadIdx.x; r < n_rows; r += ROUTE_THREADS) row_token[r] = -1;
    for (int i = threadIdx.x; i < n_rows / tile; i += ROUTE_THREADS) tile_group[i] = -1;
    __syncthreads();
    // four pairs of a thread at a time: their token ids are requested together, then their table entries (one pair
    // at a time, every pair cost two trips to memory one after the other)
    auto experts_of = [&](int base, int* e) {
        int id[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int pair = base + u * ROUTE_THREADS;
            id[u] = pair < n_pairs ? (ids ? ids[pair / top] : pair / top) : -1;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int pair = base + u * ROUTE_THREADS;
            e[u] = (id[u] >= 0 && id[u] < vocab) ? table[(size_t)id[u] * top + pair % top] : -1;
            if (e[u] >= n_experts) e[u] = -1;
        }
    };
    for (int base = threadIdx.x; base < n_pairs; base += 4 * ROUTE_THREADS) {
        int e[4];
        experts_of(base, e);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (base + u * ROUTE_THREADS >= n_pairs) break;
            if (e[u] < 0) atomicOr(error_flag, 1);
            else atomicAdd(&count[e[u]], 1);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int row = 0;
        for (int e = 0; e < n_experts; ++e) {
            first[e] = row;
            const int tiles = (count[e] + tile - 1) / tile;
            for (int i = 0; i < tiles; ++i) tile_group[row / tile + i] = e;
            row += tiles * tile;
            count[e] = 0;                        // from here on: the expert's cursor
        }
        first[n_experts] = row;
    }
    __syncthreads();
    for (int base = threadIdx.x; base < n_pairs; base += 4 * ROUTE_THREADS) {
        int e[4];
        experts_of(base, e);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int pair = base + u * ROUTE_THREADS;
            if (pair >= n_pairs) break;
            if (e[u] < 0) {
                pair_row[pair] = -1;
                continue;
            }
            const int row = first[e[u]] + atomicAdd(&count[e[u]], 1);
            pair_row[pair] = row;
            row_token[row] = pair / top;
        }
    }
}


// A 16-byte piece of a row as float32 values (exact for both storage types).
template <typename T> struct RoutePiece;
template <> struct RoutePiece<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
};
template <> struct RoutePiece<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void load(const __nv_bfloat16* p, float* out) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

// A block per token. First the router's logits, float32 sums of exact products: the block's four warps share the row's
// columns out (piece w * 32 + lane, then every 128th), each lane sums its pieces against seventeen router rows at a time
// (their loads are in flight together), a warp's lanes are added in a fixed tree and the four warps' sums in warp order,
// so a token's logits do not depend on what else is in the step. Then the first warp: the scores of the E experts in
// shared memory; a run's worth by the lanes (a run each); the worthiest runs and then the best experts by repeated
// arg-max over the warp, the lowest index winning a tie.
template <typename T>
__global__ void __launch_bounds__(128)
route_by_score_kernel(const T* __restrict__ y, int ldy, const T* __restrict__ router, int ldr, int width, int n_tokens,
                      int n_experts, int top, int groups, int keep, float weight_scale, int gate_row,
                      int* __restrict__ chosen, float* __restrict__ pair_weight, float* __restrict__ shared_scale) {
    extern __shared__ float route_smem[];        // [E] scores, [groups] worths, [4][rows] the warps' sums
    dd_launch_dependents();
    dd_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int n_rows = n_experts + (gate_row >= 0 ? 1 : 0);          // the shared unit's gate vector is one more row
    float* score = route_smem;
    float* worth = score + n_experts;
    float* part = worth + groups;
    const T* x = y + (size_t)t * ldy;
    constexpr int V = RoutePiece<T>::N, ROWS = 17;       // sixteen experts and a shared unit's gate in one pass
    const bool wide = width % V == 0 && ldy % V == 0 && ldr % V == 0 && !(((uintptr_t)y | (uintptr_t)router) & 15);
    for (int e0 = 0; e0 < n_rows; e0 += ROWS) {
        float acc[ROWS];
#pragma unroll
        for (int j = 0; j < ROWS; ++j) acc[j] = 0.f;
        if (wide) {
            for (int c = (warp * 32 + lane) * V; c < width; c += 128 * V) {
                float xv[V];
                RoutePiece<T>::load(x + c, xv);
#pragma unroll
                for (int j = 0; j < ROWS; ++j) {
                    if (e0 + j >= n_rows) break;
                    float wv[V];
                    RoutePiece<T>::load(router + (size_t)(e0 + j) * ldr + c, wv);
#pragma unroll
                    for (int i = 0; i < V; ++i) acc[j] = fmaf(xv[i], wv[i], acc[j]);
                }
            }
        } else {
            for (int c = warp * 32 + lane; c < width; c += 128) {
                const float xv = dd_to_f32(x[c]);
#pragma unroll
                for (int j = 0; j < ROWS; ++j)
                    if (e0 + j < n_rows) acc[j] = fmaf(xv, dd_to_f32(router[(size_t)(e0 + j) * ldr + c]), acc[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < ROWS; ++j) {
            const float z = dd_warp_sum(acc[j]);
            if (lane == 0 && e0 + j < n_rows) part[warp * n_rows + e0 + j] = z;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_rows; e += 128) {
        const float z = ((part[e] + part[n_rows + e]) + part[2 * n_rows + e]) + part[3 * n_rows + e];
        const float s = 1.0f / (1.0f + expf(-z));
        if (e < n_experts) score[e] = s;
        else if (shared_scale) shared_scale[t] = s;
    }
    if (threadIdx.x == 0 && shared_scale && gate_row < 0) shared_scale[t] = 1.0f;
    __syncthreads();
    if (warp) return;
    __syncwarp();
    const int per = n_experts / groups;
    if (groups > 1) {
        for (int g = lane; g < groups; g += 32) {
            float best = -1.f, second = -1.f;            // scores lie in [0, 1]
            for (int i = 0; i < per; ++i) {
                const float s = score[g * per + i];
                if (s > best) { second = best; best = s; }
                else if (s > second) second = s;
            }
            worth[g] = best + (per > 1 ? second : 0.f);
        }
        __syncwarp();
        // keep the worthiest runs: the others' scores are struck out
        for (int round = 0; round < keep; ++round) {
            float best = -1.f;
            int at = 0x7fffffff;
            for (int g = lane; g < groups; g += 32)
                if (worth[g] > best) { best = worth[g]; at = g; }
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
            }
            if (lane == 0 && at < groups) worth[at] = -2.f;     // marked as kept
            __syncwarp();
        }
        for (int e = lane; e < n_experts; e += 32)
            if (worth[e / per] != -2.f) score[e] = -1.f;
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        float best = -1.f;
        int at = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32)
            if (score[e] > best) { best = score[e]; at = e; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (lane == 0) {
            chosen[(size_t)t * top + k] = at < n_experts ? at : -1;
            pair_weight[(size_t)t * top + k] = at < n_experts ? best * weight_scale : 0.f;
            if (at < n_experts) score[at] = -1.f;
        }
        __syncwarp();
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
gather_rows_kernel(const T* __restrict__ x, const int* __restrict__ row_token, T* __restrict__ out, int width) {
    dd_launch_dependents();
    dd_grid_wait();
    const int row = blockIdx.x;
    const int t = row_token[row];
    T* o = out + (size_t)row * width;
    constexpr int V = 16 / sizeof(T);
    if (width % V == 0 && !(((uintptr_t)x | (uintptr_t)out) & 15)) {
        const uint4* src = t >= 0 ? reinterpret_cast<const uint4*>(x + (size_t)t * width) : nullptr;
        for (int c = threadIdx.x; c < width / V; c += blockDim.x)
            reinterpret_cast<uint4*>(o)[c] = src ? src[c] : make_uint4(0u, 0u, 0u, 0u);
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = t >= 0 ? x[(size_t)t * width + c] : dd_from_f32<T>(0.f);
}

template <typename T>
__global__ void __launch_bounds__(256)
gated_unit_kernel(const T* __restrict__ gate_up, int stride, T* __restrict__ out, int out_stride, int rows, int inner,
                  float limit, float alpha, int form, const float* __restrict__ row_scale) {
    dd_launch_dependents();
    dd_grid_wait();
    constexpr int V = 16 / sizeof(T);          // elements of a 16-byte piece
    const bool wide = inner % V == 0 && stride % V == 0 && out_stride % V == 0 && !(((uintptr_t)gate_up | (uintptr_t)out) & 15);
    auto unit = [&](float g, float u) { return dd_gated_value<false>(g, u, form, limit, alpha); };
    if (wide) {
        // a thread owns a piece of V neighbouring features of one row: two 16-byte loads, one 16-byte store
        const int pieces = inner / V;
        const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
        if (i >= (long long)rows * pieces) return;
        const int row = (int)(i / pieces), c = (int)(i - (long long)row * pieces) * V;
        const T* src = gate_up + (size_t)row * stride + c;
        __align__(16) T g[V], u[V], y[V];
        *reinterpret_cast<uint4*>(g) = *reinterpret_cast<const uint4*>(src);
        *reinterpret_cast<uint4*>(u) = *reinterpret_cast<const uint4*>(src + inner);
        const float by = row_scale ? row_scale[row] : 1.0f;
#pragma unroll
        for (int e = 0; e < V; ++e) y[e] = dd_from_f32<T>(unit(dd_to_f32(g[e]), dd_to_f32(u[e])) * by);
        *reinterpret_cast<uint4*>(out + (size_t)row * out_stride + c) = *reinterpret_cast<const uint4*>(y);
        return;
    }
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)rows * inner; i += (long long)gridDim.x * blockDim.x) {
        const int row = (int)(i / inner), c = (int)(i - (long long)row * inner);
        out[(size_t)row * out_stride + c] = dd_from_f32<T>(unit(dd_to_f32(gate_up[(size_t)row * stride + c]),
                                                                dd_to_f32(gate_up[(size_t)row * stride + inner + c])) *
                                                           (row_scale ? row_scale[row] : 1.0f));
    }
}

__global__ void __launch_bounds__(128)
combine_rows_kernel(const float* __restrict__ y, const int* __restrict__ pair_row, float* __restrict__ stream, int width,
                    int top, float weight, const float* __restrict__ pair_weight) {
    dd_launch_dependents();
    dd_grid_wait();
    const int t = blockIdx.x;
    // A block owns a token and a stretch of 128 x 4 (or 128) columns. The rows of eight choices are looked up first and
    // then requested together, and added in the order of the choices (one row at a time, each element cost a lookup
    // and a load one after the other: 17 us for eight tokens).
    const bool wide = width % 4 == 0 && !(((uintptr_t)y | (uintptr_t)stream) & 15);
    const int per = wide ? 4 : 1;
    const int c = (blockIdx.y * 128 + threadIdx.x) * per;
    if (c >= width) return;
    float sum[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < top; k0 += 8) {
        int row[8];
        float4 v[8];
        float by[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            row[u] = k0 + u < top ? pair_row[(size_t)t * top + k0 + u] : -1;
            by[u] = (pair_weight && k0 + u < top) ? pair_weight[(size_t)t * top + k0 + u] : 1.0f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row[u] < 0) continue;
            const float* src = y + (size_t)row[u] * width + c;
            if (wide) v[u] = *reinterpret_cast<const float4*>(src);
            else v[u].x = *src;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            sum[0] = fmaf(v[u].x, by[u], sum[0]); sum[1] = fmaf(v[u].y, by[u], sum[1]);
            sum[2] = fmaf(v[u].z, by[u], sum[2]); sum[3] = fmaf(v[u].w, by[u], sum[3]);
        }
    }
    float* dst = stream + (size_t)t * width + c;
    if (wide) {
        float4 s4 = *reinterpret_cast<float4*>(dst);
        s4.x += sum[0] * weight; s4.y += sum[1] * weight; s4.z += sum[2] * weight; s4.w += sum[3] * weight;
        *reinterpret_cast<float4*>(dst) = s4;
    } else {
        *dst += sum[0] * weight;
    }
}
}  // namespace

// n_rows: rows of the sorted buffer, a multiple of tile and at least n_tokens * top + min(n_experts, n_tokens * top)
// * (tile - 1): every expert that has a pair may waste all but one row of its last tile. A token id or a table entry out of range sets error bit 1 and leaves its pair out.
DD_API int dd_route_by_table(const int* ids, const int* table, int n_tokens, int vocab, int top, int n_experts, int tile,
                             int n_rows, int* pair_row, int* row_token, int* tile_group, int* error_flag, void* stream) {
    if (n_tokens <= 0) return 0;
    const long long n_pairs = (long long)n_tokens * top;
    if (top <= 0 || n_experts <= 0 || tile <= 0 || n_rows % tile ||
        (long long)n_rows < n_pairs + (n_pairs < n_experts ? n_pairs : (long long)n_experts) * (tile - 1))
        return dd_fail("dd_route_by_table: %d rows in tiles of %d do not hold %d tokens x %d of %d experts", n_rows, tile,
                       n_tokens, top, n_experts);
    if (n_experts > 8192) return dd_fail("dd_route_by_table: %d experts are more than a block counts", n_experts);
    dd_launch(route_by_table_kernel, dim3(1), dim3(ROUTE_THREADS), (size_t)(2 * n_experts + 1) * sizeof(int), (cudaStream_t)stream,
              ids, table, n_tokens, vocab, top, n_experts, tile, n_rows, pair_row, row_token, tile_group, error_flag);
    return dd_check_launch("dd_route_by_table");
}

// y: [n_tokens] rows of ldy elements, `width` of them the token's normed row; router: [n_experts (+ 1)] rows of ldr
// elements (the same storage type). logit = y . router row, float32 sums of exact products; score = sigmoid(logit). The
// experts form `groups` equal runs of neighbours, a run's worth is the sum of its two largest scores (of its one), only the
// `keep` worthiest runs stay eligible; the `top` largest eligible scores win. chosen: int32 [n_tokens, top] by falling
// score (-1 where fewer were eligible), pair_weight: float32 [n_tokens, top] = score * weight_scale. shared_scale (or
// null): float32 [n_tokens] = sigmoid(y . router row gate_row), 1 with gate_row < 0 (gate_row is n_experts or negative).
DD_API int dd_route_by_score(const void* y, int ldy, const void* router, int ldr, int width, int n_tokens, int n_experts,
                             int top, int groups, int keep, float weight_scale, int gate_row, int* chosen,
                             float* pair_weight, float* shared_scale, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (n_experts <= 0 || top <= 0 || top > n_experts || groups <= 0 || n_experts % groups || keep <= 0 || keep > groups ||
        (gate_row >= 0 && gate_row != n_experts) || width <= 0)
        return dd_fail("dd_route_by_score: %d of %d experts in %d groups of which %d stay, gate row %d", top, n_experts, groups, keep, gate_row);
    const size_t smem = (size_t)(n_experts + groups + 4 * (n_experts + 1)) * sizeof(float);
    if (smem > 48 * 1024) return dd_fail("dd_route_by_score: %d experts are more than a block's shared memory holds", n_experts);
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_tokens);
    if (dtype == DD_F32)
        dd_launch(route_by_score_kernel<float>, grid, dim3(128), smem, s, (const float*)y, ldy, (const float*)router, ldr, width,
                  n_tokens, n_experts, top, groups, keep, weight_scale, gate_row, chosen, pair_weight, shared_scale);
    else if (dtype == DD_BF16)
        dd_launch(route_by_score_kernel<__nv_bfloat16>, grid, dim3(128), smem, s, (const __nv_bfloat16*)y, ldy,
                  (const __nv_bfloat16*)router, ldr, width, n_tokens, n_experts, top, groups, keep, weight_scale, gate_row, chosen,
                  pair_weight, shared_scale);
    else
        return dd_fail("dd_route_by_score: unknown dtype %d", dtype);
    return dd_check_launch("dd_route_by_score");
}

DD_API int dd_gather_rows(const void* x, const int* row_token, void* out, int n_rows, int width, int dtype, void* stream) {
    if (n_rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DD_F32)
        dd_launch(gather_rows_kernel<float>, dim3(n_rows), dim3(128), 0, s, (const float*)x, row_token, (float*)out, width);
    else if (dtype == DD_BF16)
        dd_launch(gather_rows_kernel<__nv_bfloat16>, dim3(n_rows), dim3(128), 0, s, (const __nv_bfloat16*)x, row_token,
                  (__nv_bfloat16*)out, width);
    else
        return dd_fail("dd_gather_rows: unknown dtype %d", dtype);
    return dd_check_launch("dd_gather_rows");
}

// gate_up: rows of `stride` elements, the gate's `inner` values followed by the up projection's.
// form: DD_GATED_* (common.cuh); row_scale: float32 [rows] or null.
DD_API int dd_gated_unit(const void* gate_up, int stride, void* out, int out_stride, int rows, int inner, float limit,
                         float alpha, int dtype, void* stream, int form, const float* row_scale) {
    if (rows <= 0 || inner <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    // a thread takes a 16-byte piece where rows allow it, else elements in a grid-stride loop
    const int piece = dtype == DD_F32 ? 4 : 8;
    const bool wide = inner % piece == 0 && stride % piece == 0 && out_stride % piece == 0 && !(((uintptr_t)gate_up | (uintptr_t)out) & 15);
    const int grid = dd_ceil_div((long long)rows * (wide ? inner / piece : inner), 256);
    if (dtype == DD_F32)
        dd_launch(gated_unit_kernel<float>, dim3(grid), dim3(256), 0, s, (const float*)gate_up, stride, (float*)out,
                  out_stride, rows, inner, limit, alpha, form, row_scale);
    else if (dtype == DD_BF16)
        dd_launch(gated_unit_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, (const __nv_bfloat16*)gate_up, stride,
                  (__nv_bfloat16*)out, out_stride, rows, inner, limit, alpha, form, row_scale);
    else
        return dd_fail("dd_gated_unit: unknown dtype %d", dtype);
    return dd_check_launch("dd_gated_unit");
}

DD_API int dd_combine_rows(const float* y, const int* pair_row, float* stream_rows, int n_tokens, int width, int top,
                           float weight, void* stream, const float* pair_weight) {
    if (n_tokens <= 0) return 0;
    const bool wide = width % 4 == 0 && !(((uintptr_t)y | (uintptr_t)stream_rows) & 15);
    dd_launch(combine_rows_kernel, dim3(n_tokens, dd_ceil_div(width, wide ? 512 : 128)), dim3(128), 0, (cudaStream_t)stream, y, pair_row,
              stream_rows, width, top, weight, pair_weight);
    return dd_check_launch("dd_combine_rows");
}
