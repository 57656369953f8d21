// Retention: linear attention with a fixed decay per head and no softmax, over per-request state.
//
// Per head, with q_t, k_t of dk values and v_t of dv values (row views of one buffer, what a fused projection leaves):
//
//     S_t = decay * S_(t-1) + k'_t v_t^T        o_t = S_t^T q'_t
//
// where q', k' are q, k after the rotary rotation of their first 2 * n_pairs dimensions (as in rotary.cu; the two
// layouts) and k' is also multiplied by key_scale. S [dk, dv] is float32 and lives in the request's state slot,
// stored column by column ([slots, heads, dv, dk]: the dk values that one output column reads lie together). Rotation,
// products, sums and state are float32 whatever the storage type of the projections; nothing is rounded between the
// projection's output and o.
//
// dd_retention runs the recurrence for every entry of a step from the state earlier steps left, token by token in
// position order, so a prompt's portion and a single decoded token take the same arithmetic in the same order: the
// result does not depend on how a prompt was cut. Column j of o depends on column j of S only, so a block owns
// (entry, head, a slice of 32 columns): 8 warps x 4 columns, a lane the rows lane, lane + 32, ... of its 4 columns in
// registers. Tokens are staged through shared memory 16 at a time, rotated on the way. o goes to float32 scratch.
//
// dd_retention_finish then divides every head's o by its root mean square (eps inside the root, no weight), multiplies
// by silu(gate) and rounds to the storage type: the operand of the output projection.
#include "common.cuh"

namespace {
constexpr int THREADS = 256, COLS = 32, COLS_PER_WARP = 4, CHUNK = 16;

struct RetentionArgs {
    int stride;                  // row stride of q, k, v (elements)
    const int* positions;        // [tokens]
    const int* entry_start;      // [entries + 1]
    const int* entry_slot;       // [entries]
    const float* freqs;          // [n_pairs]
    const float* decay;          // [heads]
    float* state;                // [slots, heads, dv, dk]
    float* o;                    // [tokens, heads * dv]
    int heads, dk, dv, n_pairs, interleaved, n_slots;
    float key_scale;
    int* error_flag;
};

// R: rows a lane owns (dk <= 32 R)
template <typename T, int R>
__global__ void __launch_bounds__(THREADS)
retention_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const RetentionArgs a) {
    extern __shared__ float staged[];            // [CHUNK][dk] rotated queries, [CHUNK][dk] rotated scaled keys, [CHUNK][COLS] values
    float* qs = staged;
    float* ks = staged + CHUNK * a.dk;
    float* vs = ks + CHUNK * a.dk;
    dd_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slices = (a.dv + COLS - 1) / COLS;
    const int slice = blockIdx.x % slices;
    const int h = (blockIdx.x / slices) % a.heads;
    const int e = blockIdx.x / (slices * a.heads);
    const int t0 = a.entry_start[e], t1 = a.entry_start[e + 1];
    const int slot = a.entry_slot[e];
    const float decay = a.decay[h];
    if (slot < 0 || slot >= a.n_slots) {
        if (threadIdx.x == 0) atomicOr(a.error_flag, 1);
        return;
    }
    const int col0 = slice * COLS + warp * COLS_PER_WARP;
    // the state is an earlier step's (or zeros): it is in registers before the projection before this kernel has finished
    float S[R][COLS_PER_WARP];
    float* state = a.state + ((size_t)slot * a.heads + h) * (size_t)a.dv * a.dk;
#pragma unroll
    for (int c = 0; c < COLS_PER_WARP; ++c)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = lane + 32 * r;
            S[r][c] = (col0 + c < a.dv && row < a.dk) ? state[(size_t)(col0 + c) * a.dk + row] : 0.f;
        }
    dd_grid_wait();
    const int half = a.n_pairs;
    for (int base = t0; base < t1; base += CHUNK) {
        const int n = min(CHUNK, t1 - base);
        __syncthreads();                         // the chunk before has been read
        for (int idx = threadIdx.x; idx < n * a.dk; idx += THREADS) {
            const int tt = idx / a.dk, i = idx - tt * a.dk;
            const size_t at = (size_t)(base + tt) * a.stride + (size_t)h * a.dk;
            float qv = dd_to_f32(q[at + i]), kv = dd_to_f32(k[at + i]);
            if (i < 2 * half) {
                // the pair this dimension belongs to, whether it is the pair's first member, and its partner
                const int pair = a.interleaved ? i >> 1 : (i < half ? i : i - half);
                const bool first = a.interleaved ? !(i & 1) : i < half;
                const int other = a.interleaved ? i ^ 1 : (first ? i + half : i - half);
                float sn, cs;
                sincosf((float)a.positions[base + tt] * a.freqs[pair], &sn, &cs);
                const float qo = dd_to_f32(q[at + other]), ko = dd_to_f32(k[at + other]);
                qv = first ? qv * cs - qo * sn : qv * cs + qo * sn;
                kv = first ? kv * cs - ko * sn : kv * cs + ko * sn;
            }
            qs[idx] = qv;
            ks[idx] = kv * a.key_scale;
        }
        for (int idx = threadIdx.x; idx < n * COLS; idx += THREADS) {
            const int tt = idx / COLS, j = slice * COLS + (idx % COLS);
            vs[idx] = j < a.dv ? dd_to_f32(v[(size_t)(base + tt) * a.stride + (size_t)h * a.dv + j]) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            float kk[R], qq[R], vv[COLS_PER_WARP], o[COLS_PER_WARP];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int row = lane + 32 * r;
                kk[r] = row < a.dk ? ks[tt * a.dk + row] : 0.f;
                qq[r] = row < a.dk ? qs[tt * a.dk + row] : 0.f;
            }
#pragma unroll
            for (int c = 0; c < COLS_PER_WARP; ++c) {
                vv[c] = vs[tt * COLS + warp * COLS_PER_WARP + c];
                o[c] = 0.f;
            }
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int c = 0; c < COLS_PER_WARP; ++c) {
                    S[r][c] = fmaf(decay, S[r][c], kk[r] * vv[c]);
                    o[c] = fmaf(S[r][c], qq[r], o[c]);
                }
            // four columns summed over the 32 lanes in six exchanges: halves of the warp trade columns, then quarters,
            // then the eight lanes that hold one column's parts are added
            const bool upper = lane & 16;
            float keep0 = upper ? o[2] : o[0], keep1 = upper ? o[3] : o[1];
            keep0 += __shfl_xor_sync(0xffffffffu, upper ? o[0] : o[2], 16);
            keep1 += __shfl_xor_sync(0xffffffffu, upper ? o[1] : o[3], 16);
            const bool odd = lane & 8;
            float sum = odd ? keep1 : keep0;
            sum += __shfl_xor_sync(0xffffffffu, odd ? keep0 : keep1, 8);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            const int col = col0 + (upper ? 2 : 0) + (odd ? 1 : 0);
            if (!(lane & 7) && col < a.dv) a.o[(size_t)(base + tt) * a.heads * a.dv + (size_t)h * a.dv + col] = sum;
        }
    }
#pragma unroll
    for (int c = 0; c < COLS_PER_WARP; ++c)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = lane + 32 * r;
            if (col0 + c < a.dv && row < a.dk) state[(size_t)(col0 + c) * a.dk + row] = S[r][c];
        }
}

template <typename T>
__global__ void __launch_bounds__(128)
retention_finish_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_stride, T* __restrict__ out,
                        int out_stride, int n_tokens, int heads, int dv, float eps) {
    dd_launch_dependents();
    dd_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)n_tokens * heads) return;
    const int t = (int)(item / heads), h = (int)(item % heads);
    const float* row = o + (size_t)t * heads * dv + (size_t)h * dv;
    float sq = 0.f;
    for (int c = lane; c < dv; c += 32) sq += row[c] * row[c];
    sq = dd_warp_sum(sq);
    const float r = 1.0f / sqrtf(sq / (float)dv + eps);
    const T* g = gate + (size_t)t * gate_stride + (size_t)h * dv;
    T* dst = out + (size_t)t * out_stride + (size_t)h * dv;
    for (int c = lane; c < dv; c += 32) {
        const float z = dd_to_f32(g[c]);
        dst[c] = dd_from_f32<T>(row[c] * r * (z / (1.0f + expf(-z))));
    }
}

template <typename T>
int launch_retention(const void* q, const void* k, const void* v, const RetentionArgs& a, int n_entries, cudaStream_t s) {
    const int slices = (a.dv + COLS - 1) / COLS;
    const long long blocks = (long long)n_entries * a.heads * slices;
    if (blocks > 0x7fffffffLL) return dd_fail("dd_retention: %d entries x %d heads x %d slices are too many blocks", n_entries, a.heads, slices);
    const size_t smem = (size_t)CHUNK * (2 * a.dk + COLS) * sizeof(float);
#define DD_RETENTION(R)                                                                                              \
    dd_launch(retention_kernel<T, R>, dim3((unsigned)blocks), dim3(THREADS), smem, s, (const T*)q, (const T*)k, (const T*)v, a)
    if (a.dk <= 32) DD_RETENTION(1);
    else if (a.dk <= 64) DD_RETENTION(2);
    else if (a.dk <= 128) DD_RETENTION(4);
    else DD_RETENTION(8);
#undef DD_RETENTION
    return dd_check_launch("dd_retention");
}
}  // namespace

// q, k: [tokens] rows of `stride` elements with `heads` heads of dk; v likewise with heads of dv. The tokens of entry e are
// rows entry_start[e] .. entry_start[e + 1] - 1 at consecutive positions; its state is row entry_slot[e] of `state`
// (float32 [n_slots, heads, dv, dk]), read and written. decay: float32 [heads] on the device. freqs: float32 [n_pairs]
// or null with n_pairs == 0. o: float32 [tokens, heads * dv]. A slot outside the state sets error bit 1.
DD_API int dd_retention(const void* q, const void* k, const void* v, int stride, const int* positions, const int* entry_start,
                        const int* entry_slot, int n_entries, const float* freqs, int n_pairs, int interleaved,
                        const float* decay, float key_scale, float* state, int n_slots, float* o, int heads, int dk, int dv,
                        int dtype, int* error_flag, void* stream) {
    if (n_entries <= 0) return 0;
    if (heads <= 0 || dk <= 0 || dk > 256 || dv <= 0)
        return dd_fail("dd_retention: %d heads of %d (at most 256) and %d are not supported", heads, dk, dv);
    if (n_pairs < 0 || 2 * n_pairs > dk || (n_pairs > 0 && !freqs)) return dd_fail("dd_retention: %d pairs do not fit a head of %d", n_pairs, dk);
    RetentionArgs a;
    a.stride = stride; a.positions = positions; a.entry_start = entry_start; a.entry_slot = entry_slot; a.freqs = freqs;
    a.decay = decay; a.state = state; a.o = o; a.heads = heads; a.dk = dk; a.dv = dv; a.n_pairs = n_pairs;
    a.interleaved = interleaved; a.n_slots = n_slots; a.key_scale = key_scale; a.error_flag = error_flag;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DD_F32) return launch_retention<float>(q, k, v, a, n_entries, s);
    if (dtype == DD_BF16) return launch_retention<__nv_bfloat16>(q, k, v, a, n_entries, s);
    return dd_fail("dd_retention: unknown dtype %d", dtype);
}

// o: float32 [tokens, heads * dv]; gate: rows of gate_stride elements with heads * dv values; out likewise (out_stride).
DD_API int dd_retention_finish(const float* o, const void* gate, int gate_stride, void* out, int out_stride, int n_tokens,
                               int heads, int dv, float eps, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int grid = dd_ceil_div((long long)n_tokens * heads, 4);
    if (dtype == DD_F32)
        dd_launch(retention_finish_kernel<float>, dim3(grid), dim3(128), 0, s, o, (const float*)gate, gate_stride, (float*)out,
                  out_stride, n_tokens, heads, dv, eps);
    else if (dtype == DD_BF16)
        dd_launch(retention_finish_kernel<__nv_bfloat16>, dim3(grid), dim3(128), 0, s, o, (const __nv_bfloat16*)gate, gate_stride,
                  (__nv_bfloat16*)out, out_stride, n_tokens, heads, dv, eps);
    else
        return dd_fail("dd_retention_finish: unknown dtype %d", dtype);
    return dd_check_launch("dd_retention_finish");
}
