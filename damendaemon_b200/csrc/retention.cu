// Retention: linear attention with a fixed decay per head and no softmax, over per-request state.
//
// Per head, with q_t, k_t of dk values and v_t of dv values (row views of one buffer, what a fused projection leaves):
//
//     S_t = decay * S_(t-1) + k'_t v_t^T        o_t = S_t^T q'_t
//
// where q', k' are q, k after the rotary rotation of their first 2 * n_pairs dimensions (as in rotary.cu; the two
// layouts) and k' is also multiplied by key_scale. S [dk, dv] is float32 and lives in the request's state slot,
// stored column by column ([slots, heads, dv, dkp] with dkp = dk rounded up to 4: the values that one output column reads
// lie together, and a thread's four rows are one 16-byte piece). Rotation, products, sums and state are float32 whatever
// the storage type of the projections; nothing is rounded between the projection's output and o.
//
// dd_retention runs the recurrence for every entry of a step from the state earlier steps left, token by token in
// position order, so a prompt's portion and a single decoded token take the same arithmetic in the same order: the
// result does not depend on how a prompt was cut. Column j of o depends on column j of S only, so a block owns
// (entry, head, a slice of columns). A thread keeps R = 8 rows of one column in registers; L neighbouring lanes share a
// column (L a power of two, dk <= R L), so a warp holds 32 / L columns and a column's read-out is summed over L lanes in
// log2 L exchanges. The tokens of an entry come one after the other; only entries, heads, columns and rows run side by
// side, and a scheduler needs several warps to hide the shared-memory and exchange latencies of each, so R trades
// instructions against warps (measured at 25 heads of 64 x 64: a warp spends 83 instructions a token with 4 rows a thread
// and 133 with 16, for a quarter of the warps; two prompts of 1,024 tokens took the same time either way, a decode step
// of 64 requests 33 and 21 us; 8 rows lie between). A block has 8, 4, 2 or 1 warps: the fewest columns a block that
// still gives the GPU two blocks an SM. o goes to float32 scratch. With portions the recurrence is launched in plain
// stream order and lets its successor start only when its tokens are done: started early, its few long-running blocks
// went wherever the kernel before had just freed room, several to an SM, and stayed there (two prompts of 1,024 tokens:
// 613 against 312 us).
//
// Two ways in, one arithmetic (the rotation and the recurrence are the same functions, written with explicit
// fused-multiply-add intrinsics so that both paths round alike). A step of single tokens: the block rotates its token
// itself while staging it (one launch). A step with prompt portions: dd_retention first writes rotated q, scaled rotated
// k and v as float32 rows into scratch (retention_prepare_kernel: a block a token, its cosines and sines computed once
// for all heads), so that the narrow blocks of the recurrence do not each repeat the rotation; they then stage their
// chunks by cp.async into two buffers in turn, the next chunk on its way while this one is computed, and run four
// tokens' read-outs side by side (a token's state update depends on the token before, its read-out's sum on nothing
// that follows).
//
// dd_retention_finish then divides every head's o by its root mean square (eps inside the root, no weight), multiplies
// by silu(gate) and rounds to the storage type: the operand of the output projection.
#include "common.cuh"

namespace {
constexpr int CHUNK = 16, PREP_WARPS = 8;

struct RetentionArgs {
    int stride;                  // row stride of q, k, v (elements)
    const int* positions;        // [tokens]
    const int* entry_start;      // [entries + 1]
    const int* entry_slot;       // [entries]
    const float* freqs;          // [n_pairs]
    const float* decay;          // [heads]
    float* state;                // [slots, heads, dv, dkp]
    float* o;                    // [tokens, heads * dv]
    int heads, dk, dv, n_pairs, interleaved, n_slots;
    float key_scale;
    int* error_flag;
    const float* prepared;       // [tokens, heads, 2 dkp + dvp]: rotated q, rotated scaled k, v as float32, or null
    int dkp, dvp, chunk;         // dk and dv rounded up to 4; tokens staged at a time
};

// (a, b) -> (a c - b s, b c + a s), rounded the same way wherever it is compiled
__device__ __forceinline__ void rotate_pair(float a, float b, float cs, float sn, float& oa, float& ob) {
    oa = __fmaf_rn(a, cs, -__fmul_rn(b, sn));
    ob = __fmaf_rn(b, cs, __fmul_rn(a, sn));
}

// One token of the recurrence for a thread's R rows of its column: S = decay S + k v, and the thread's part of S^T q
// (two running sums, so that the chain of dependent additions is half as long).
template <int R>
__device__ __forceinline__ float retention_token(float (&S)[R], const float* tok_q, const float* tok_k, float v, float decay) {
    float even = 0.f, odd = 0.f;
#pragma unroll
    for (int r = 0; r < R; r += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(tok_k + r);
        const float4 q4 = *reinterpret_cast<const float4*>(tok_q + r);
        S[r] = __fmaf_rn(decay, S[r], __fmul_rn(k4.x, v));
        S[r + 1] = __fmaf_rn(decay, S[r + 1], __fmul_rn(k4.y, v));
        S[r + 2] = __fmaf_rn(decay, S[r + 2], __fmul_rn(k4.z, v));
        S[r + 3] = __fmaf_rn(decay, S[r + 3], __fmul_rn(k4.w, v));
        even = __fmaf_rn(S[r], q4.x, even);
        odd = __fmaf_rn(S[r + 1], q4.y, odd);
        even = __fmaf_rn(S[r + 2], q4.z, even);
        odd = __fmaf_rn(S[r + 3], q4.w, odd);
    }
    return even + odd;
}

// The sum over the L neighbouring lanes of a column; every one of them gets it.
template <int L>
__device__ __forceinline__ float column_sum(float part) {
#pragma unroll
    for (int o = L / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    return part;
}

__device__ __forceinline__ void copy16_async(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// R: rows a thread holds; L: lanes that share a column (dk <= R L); WARPS: warps of a block, each with 32 / L columns;
// PREPARED: the tokens come rotated, as float32 rows, from a.prepared, else from q, k, v and are rotated here.
// A staged token in shared memory: [R L] rotated q (zeros beyond dk), [R L] rotated scaled k, [COLS] this block's v.
template <typename T, int R, int L, int WARPS, bool PREPARED>
__global__ void __launch_bounds__(WARPS * 32)
retention_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const RetentionArgs a) {
    constexpr int THREADS = WARPS * 32, PER_WARP = 32 / L, COLS = WARPS * PER_WARP, DKS = R * L;
    constexpr int PER_TOKEN = 2 * DKS + (COLS + 3) / 4 * 4;
    extern __shared__ __align__(16) float staged[];            // [chunk][PER_TOKEN], twice when PREPARED
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
        dd_launch_dependents();
        return;
    }
    const int in_block = warp * PER_WARP + lane / L;           // this thread's column within the block's slice
    const int col = slice * COLS + in_block;
    const int row0 = (lane % L) * R;
    // the state is an earlier step's (or zeros): it is in registers before the projection before this kernel has finished
    float S[R];
    const bool holds = col < a.dv && row0 < a.dkp;             // rows from dk to dkp are padding that stays zero
    float4* state = reinterpret_cast<float4*>(a.state + (((size_t)slot * a.heads + h) * a.dv + min(col, a.dv - 1)) * (size_t)a.dkp +
                                              min(row0, a.dkp - 4));
#pragma unroll
    for (int i = 0; i < R / 4; ++i) {
        const float4 s4 = holds && row0 + 4 * i < a.dkp ? state[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        S[4 * i] = s4.x; S[4 * i + 1] = s4.y; S[4 * i + 2] = s4.z; S[4 * i + 3] = s4.w;
    }
    const int buffers = PREPARED ? 2 : 1;
    // rows beyond dk never change: zeroed once (copies and the staging below write [0, dkp) and [0, dk) only, and the
    // prepared rows hold zeros from dk to dkp)
    for (int idx = threadIdx.x; idx < buffers * a.chunk * 2 * DKS; idx += THREADS) {
        const int tt = idx / (2 * DKS), i = idx - tt * 2 * DKS;
        if ((i < DKS ? i : i - DKS) >= a.dk) staged[tt * PER_TOKEN + i] = 0.f;
    }
    dd_grid_wait();
    const int half = a.n_pairs;
    const int prepared_row = 2 * a.dkp + a.dvp;
    auto request = [&](int base, float* buffer) {             // PREPARED: a chunk's tokens by 16-byte copies
        const int n = min(a.chunk, t1 - base);
        const int q_pieces = a.dkp / 4, pieces = 2 * q_pieces + (COLS + 3) / 4;
        // a warp asks for every WARPS-th token of the chunk, a lane for every 32nd piece of it
        for (int tt = warp; tt < n; tt += WARPS) {
            const float* src = a.prepared + ((size_t)(base + tt) * a.heads + h) * prepared_row;
            float* dst = buffer + tt * PER_TOKEN;
            for (int piece = lane; piece < pieces; piece += 32) {
                if (piece < q_pieces) {
                    copy16_async(dst + 4 * piece, src + 4 * piece);
                } else if (piece < 2 * q_pieces) {
                    copy16_async(dst + DKS + 4 * (piece - q_pieces), src + a.dkp + 4 * (piece - q_pieces));
                } else {
                    const int c = 4 * (piece - 2 * q_pieces);
                    if (slice * COLS + c < a.dvp) copy16_async(dst + 2 * DKS + c, src + 2 * a.dkp + slice * COLS + c);
                    else *reinterpret_cast<float4*>(dst + 2 * DKS + c) = make_float4(0.f, 0.f, 0.f, 0.f);      // columns this head does not have
                }
            }
        }
        copies_commit();
    };
    if (PREPARED && t0 < t1) request(t0, staged);
    int turn = 0;
    for (int base = t0; base < t1; base += a.chunk) {
        const int n = min(a.chunk, t1 - base);
        float* now = staged + turn * a.chunk * PER_TOKEN;
        if (PREPARED) {
            if (base + a.chunk < t1) {
                request(base + a.chunk, staged + (turn ^ 1) * a.chunk * PER_TOKEN);
                copies_wait<1>();
            } else {
                copies_wait<0>();
            }
            turn ^= 1;
        } else {
            __syncthreads();                     // the chunk before has been read
            // an item is a pair of rotated dimensions (one cosine and sine serve the query's and the key's pair) or one of
            // the dimensions behind them
            const int per_token = a.dk - half;
            for (int idx = threadIdx.x; idx < n * per_token; idx += THREADS) {
                const int tt = idx / per_token, item = idx - tt * per_token;
                const size_t at = (size_t)(base + tt) * a.stride + (size_t)h * a.dk;
                float* qrow = now + tt * PER_TOKEN;
                float* krow = qrow + DKS;
                if (item < half) {
                    const int ia = a.interleaved ? 2 * item : item, ib = a.interleaved ? 2 * item + 1 : item + half;
                    float sn, cs, qa, qb, ka, kb;
                    sincosf((float)a.positions[base + tt] * a.freqs[item], &sn, &cs);
                    rotate_pair(dd_to_f32(q[at + ia]), dd_to_f32(q[at + ib]), cs, sn, qa, qb);
                    rotate_pair(dd_to_f32(k[at + ia]), dd_to_f32(k[at + ib]), cs, sn, ka, kb);
                    qrow[ia] = qa;
                    qrow[ib] = qb;
                    krow[ia] = __fmul_rn(ka, a.key_scale);
                    krow[ib] = __fmul_rn(kb, a.key_scale);
                } else {
                    const int i = item + half;
                    qrow[i] = dd_to_f32(q[at + i]);
                    krow[i] = __fmul_rn(dd_to_f32(k[at + i]), a.key_scale);
                }
            }
            for (int idx = threadIdx.x; idx < n * COLS; idx += THREADS) {
                const int tt = idx / COLS, c = idx - tt * COLS, j = slice * COLS + c;
                now[tt * PER_TOKEN + 2 * DKS + c] = j < a.dv ? dd_to_f32(v[(size_t)(base + tt) * a.stride + (size_t)h * a.dv + j]) : 0.f;
            }
        }
        __syncthreads();
        // four tokens at a time without a branch between them: their loads and sums overlap (a token's state update
        // waits for the token before, nothing else does)
        const float* tq = now + row0;
        const float* tv = now + 2 * DKS + in_block;
        float* out = a.o + ((size_t)base * a.heads + h) * a.dv + col;
        const size_t step = (size_t)a.heads * a.dv;
        const bool writer = lane % L == 0 && col < a.dv;
        int tt = 0;
        for (; tt + 4 <= n; tt += 4) {
            float p0 = retention_token<R>(S, tq, tq + DKS, tv[0], decay);
            float p1 = retention_token<R>(S, tq + PER_TOKEN, tq + PER_TOKEN + DKS, tv[PER_TOKEN], decay);
            float p2 = retention_token<R>(S, tq + 2 * PER_TOKEN, tq + 2 * PER_TOKEN + DKS, tv[2 * PER_TOKEN], decay);
            float p3 = retention_token<R>(S, tq + 3 * PER_TOKEN, tq + 3 * PER_TOKEN + DKS, tv[3 * PER_TOKEN], decay);
            p0 = column_sum<L>(p0);
            p1 = column_sum<L>(p1);
            p2 = column_sum<L>(p2);
            p3 = column_sum<L>(p3);
            if (writer) {
                out[0] = p0;
                out[step] = p1;
                out[2 * step] = p2;
                out[3 * step] = p3;
            }
            tq += 4 * PER_TOKEN;
            tv += 4 * PER_TOKEN;
            out += 4 * step;
        }
        for (; tt < n; ++tt) {
            const float p = column_sum<L>(retention_token<R>(S, tq, tq + DKS, tv[0], decay));
            if (writer) out[0] = p;
            tq += PER_TOKEN;
            tv += PER_TOKEN;
            out += step;
        }
        if (PREPARED) __syncthreads();           // this buffer is the target of the next request but one
    }
    dd_launch_dependents();
#pragma unroll
    for (int i = 0; i < R / 4; ++i)
        if (holds && row0 + 4 * i < a.dkp) state[i] = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
}

// Rotated q, rotated scaled k and v of every (token, head) as float32 rows [2 dkp + dvp] (dimensions beyond dk and dv
// zeroed). A block owns a token and a share of its heads; the token's cosines and sines are computed once.
template <typename T>
__global__ void __launch_bounds__(PREP_WARPS * 32)
retention_prepare_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const RetentionArgs a,
                         float* __restrict__ prepared, int heads_per_block) {
    extern __shared__ float table[];             // [n_pairs] cosines, [n_pairs] sines
    dd_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x, half = a.n_pairs;
    const float p = (float)a.positions[t];
    for (int i = threadIdx.x; i < half; i += PREP_WARPS * 32) sincosf(p * a.freqs[i], &table[half + i], &table[i]);
    __syncthreads();
    dd_grid_wait();
    const int row_floats = 2 * a.dkp + a.dvp;
    const int h_end = min(a.heads, (int)(blockIdx.y + 1) * heads_per_block);
    for (int h = blockIdx.y * heads_per_block + warp; h < h_end; h += PREP_WARPS) {
        const size_t at = (size_t)t * a.stride + (size_t)h * a.dk;
        float* qrow = prepared + ((size_t)t * a.heads + h) * row_floats;
        float* krow = qrow + a.dkp;
        for (int item = lane; item < a.dk - half; item += 32) {
            if (item < half) {
                const int ia = a.interleaved ? 2 * item : item, ib = a.interleaved ? 2 * item + 1 : item + half;
                float qa, qb, ka, kb;
                rotate_pair(dd_to_f32(q[at + ia]), dd_to_f32(q[at + ib]), table[item], table[half + item], qa, qb);
                rotate_pair(dd_to_f32(k[at + ia]), dd_to_f32(k[at + ib]), table[item], table[half + item], ka, kb);
                qrow[ia] = qa;
                qrow[ib] = qb;
                krow[ia] = __fmul_rn(ka, a.key_scale);
                krow[ib] = __fmul_rn(kb, a.key_scale);
            } else {
                const int i = item + half;
                qrow[i] = dd_to_f32(q[at + i]);
                krow[i] = __fmul_rn(dd_to_f32(k[at + i]), a.key_scale);
            }
        }
        for (int i = a.dk + lane; i < a.dkp; i += 32) qrow[i] = krow[i] = 0.f;
        const T* vrow = v + (size_t)t * a.stride + (size_t)h * a.dv;
        for (int c = lane; c < a.dvp; c += 32) qrow[2 * a.dkp + c] = c < a.dv ? dd_to_f32(vrow[c]) : 0.f;
    }
}

// A warp owns a (token, head): the head's o in registers (PER values a lane), one pass.
template <typename T, int PER>
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
    const T* g = gate + (size_t)t * gate_stride + (size_t)h * dv;
    float x[PER], z[PER];
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = lane + 32 * i;
        x[i] = c < dv ? row[c] : 0.f;
        z[i] = c < dv ? dd_to_f32(g[c]) : 0.f;
        sq += x[i] * x[i];
    }
    sq = dd_warp_sum(sq);
    const float r = 1.0f / sqrtf(sq / (float)dv + eps);
    T* dst = out + (size_t)t * out_stride + (size_t)h * dv;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) dst[c] = dd_from_f32<T>(x[i] * r * (z[i] / (1.0f + expf(-z[i]))));
    }
}

template <typename T, int R, int L, int WARPS>
int launch_retention_sized(const void* q, const void* k, const void* v, const RetentionArgs& a, long long blocks, cudaStream_t s) {
    const int per_token = 2 * R * L + (WARPS * (32 / L) + 3) / 4 * 4;
    const size_t smem = (size_t)(a.prepared ? 2 : 1) * a.chunk * per_token * sizeof(float);
    if (a.prepared)      // few blocks that each walk a whole entry: in stream order, so that they spread over all SMs
        dd_launch_in_order(retention_kernel<T, R, L, WARPS, true>, dim3((unsigned)blocks), dim3(WARPS * 32), smem, s, (const T*)q, (const T*)k, (const T*)v, a);
    else
        dd_launch(retention_kernel<T, R, L, WARPS, false>, dim3((unsigned)blocks), dim3(WARPS * 32), smem, s, (const T*)q, (const T*)k, (const T*)v, a);
    return dd_check_launch("dd_retention");
}

template <typename T, int R, int L>
int launch_retention_lanes(const void* q, const void* k, const void* v, const RetentionArgs& a, int n_entries, int sms, cudaStream_t s) {
    // the widest block that still gives every SM two blocks; with few entries and heads, narrower ones (of at least four
    // columns: a block's columns of v are copied in 16-byte pieces, which must start on a multiple of four)
    int warps = 8;
    const int least = 32 / L >= 4 ? 1 : 4 / (32 / L);
    auto blocks_with = [&](int w) { return (long long)n_entries * a.heads * ((a.dv + w * (32 / L) - 1) / (w * (32 / L))); };
    while (warps > least && blocks_with(warps) < 2LL * sms) warps >>= 1;
    const long long blocks = blocks_with(warps);
    if (blocks > 0x7fffffffLL) return dd_fail("dd_retention: %d entries x %d heads of %d columns are too many blocks", n_entries, a.heads, a.dv);
    if (warps == 8) return launch_retention_sized<T, R, L, 8>(q, k, v, a, blocks, s);
    if (warps == 4) return launch_retention_sized<T, R, L, 4>(q, k, v, a, blocks, s);
    if (warps == 2) return launch_retention_sized<T, R, L, 2>(q, k, v, a, blocks, s);
    return launch_retention_sized<T, R, L, 1>(q, k, v, a, blocks, s);
}

template <typename T>
int launch_retention(const void* q, const void* k, const void* v, RetentionArgs a, int n_entries, int n_tokens, float* scratch,
                     cudaStream_t s) {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    a.prepared = nullptr;
    if (scratch && n_tokens > n_entries) {
        // a step with portions: rotate once for all the narrow blocks of the recurrence
        int groups = dd_ceil_div(2 * sms, n_tokens);
        if (groups > dd_ceil_div(a.heads, PREP_WARPS)) groups = dd_ceil_div(a.heads, PREP_WARPS);
        if (groups < 1) groups = 1;
        const int heads_per_block = dd_ceil_div(a.heads, groups);
        dd_launch(retention_prepare_kernel<T>, dim3(n_tokens, dd_ceil_div(a.heads, heads_per_block)), dim3(PREP_WARPS * 32),
                  2 * (size_t)a.n_pairs * sizeof(float), s, (const T*)q, (const T*)k, (const T*)v, a, scratch, heads_per_block);
        if (int e = dd_check_launch("dd_retention (prepare)")) return e;
        a.prepared = scratch;
    }
    // eight rows a thread and as many lanes a column as hold dk (a power of two)
    if (a.dk <= 4) return launch_retention_lanes<T, 4, 1>(q, k, v, a, n_entries, sms, s);
    if (a.dk <= 8) return launch_retention_lanes<T, 8, 1>(q, k, v, a, n_entries, sms, s);
    if (a.dk <= 16) return launch_retention_lanes<T, 8, 2>(q, k, v, a, n_entries, sms, s);
    if (a.dk <= 32) return launch_retention_lanes<T, 8, 4>(q, k, v, a, n_entries, sms, s);
    if (a.dk <= 64) return launch_retention_lanes<T, 8, 8>(q, k, v, a, n_entries, sms, s);
    if (a.dk <= 128) return launch_retention_lanes<T, 8, 16>(q, k, v, a, n_entries, sms, s);
    return launch_retention_lanes<T, 8, 32>(q, k, v, a, n_entries, sms, s);
}
}  // namespace

// q, k: [tokens] rows of `stride` elements with `heads` heads of dk; v likewise with heads of dv. The tokens of entry e are
// rows entry_start[e] .. entry_start[e + 1] - 1 at consecutive positions; its state is row entry_slot[e] of `state`
// (float32 [n_slots, heads, dv, roundup(dk, 4)]; zeros for a new request), read and written. decay: float32 [heads] on the device. freqs: float32 [n_pairs]
// or null with n_pairs == 0. o: float32 [tokens, heads * dv]. A slot outside the state sets error bit 1. scratch: float32
// [n_tokens, heads, 2 * roundup(dk, 4) + roundup(dv, 4)], 16-byte aligned, wanted when an entry brings more than one token
// (n_tokens > n_entries), may be null otherwise.
DD_API int dd_retention(const void* q, const void* k, const void* v, int stride, const int* positions, const int* entry_start,
                        const int* entry_slot, int n_entries, const float* freqs, int n_pairs, int interleaved,
                        const float* decay, float key_scale, float* state, int n_slots, float* o, int heads, int dk, int dv,
                        int dtype, int* error_flag, void* stream, int n_tokens, float* scratch) {
    if (n_entries <= 0) return 0;
    if (heads <= 0 || dk <= 0 || dk > 256 || dv <= 0)
        return dd_fail("dd_retention: %d heads of %d (at most 256) and %d are not supported", heads, dk, dv);
    if (n_pairs < 0 || 2 * n_pairs > dk || (n_pairs > 0 && !freqs)) return dd_fail("dd_retention: %d pairs do not fit a head of %d", n_pairs, dk);
    if ((scratch && ((uintptr_t)scratch & 15)) || ((uintptr_t)state & 15)) return dd_fail("dd_retention: scratch and state must be 16-byte aligned");
    if (n_tokens > n_entries && !scratch) return dd_fail("dd_retention: a step with portions (%d tokens of %d entries) needs scratch", n_tokens, n_entries);
    RetentionArgs a;
    a.stride = stride; a.positions = positions; a.entry_start = entry_start; a.entry_slot = entry_slot; a.freqs = freqs;
    a.decay = decay; a.state = state; a.o = o; a.heads = heads; a.dk = dk; a.dv = dv; a.n_pairs = n_pairs;
    a.interleaved = interleaved; a.n_slots = n_slots; a.key_scale = key_scale; a.error_flag = error_flag;
    a.prepared = nullptr; a.dkp = (dk + 3) / 4 * 4; a.dvp = (dv + 3) / 4 * 4; a.chunk = dk <= 128 ? CHUNK : CHUNK / 2;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DD_F32) return launch_retention<float>(q, k, v, a, n_entries, n_tokens, scratch, s);
    if (dtype == DD_BF16) return launch_retention<__nv_bfloat16>(q, k, v, a, n_entries, n_tokens, scratch, s);
    return dd_fail("dd_retention: unknown dtype %d", dtype);
}

// o: float32 [tokens, heads * dv]; gate: rows of gate_stride elements with heads * dv values; out likewise (out_stride).
DD_API int dd_retention_finish(const float* o, const void* gate, int gate_stride, void* out, int out_stride, int n_tokens,
                               int heads, int dv, float eps, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (dv <= 0 || dv > 1024) return dd_fail("dd_retention_finish: a value head of %d is not supported (at most 1024)", dv);
    cudaStream_t s = (cudaStream_t)stream;
    const int grid = dd_ceil_div((long long)n_tokens * heads, 4);
#define DD_FINISH(T, PER)                                                                                                 \
    dd_launch(retention_finish_kernel<T, PER>, dim3(grid), dim3(128), 0, s, o, (const T*)gate, gate_stride, (T*)out, out_stride, \
              n_tokens, heads, dv, eps)
#define DD_FINISH_SIZED(T)                                                     \
    do {                                                                       \
        if (dv <= 32) DD_FINISH(T, 1);                                         \
        else if (dv <= 64) DD_FINISH(T, 2);                                    \
        else if (dv <= 128) DD_FINISH(T, 4);                                   \
        else if (dv <= 256) DD_FINISH(T, 8);                                   \
        else DD_FINISH(T, 32);                                                 \
    } while (0)
    if (dtype == DD_F32) DD_FINISH_SIZED(float);
    else if (dtype == DD_BF16) DD_FINISH_SIZED(__nv_bfloat16);
    else return dd_fail("dd_retention_finish: unknown dtype %d", dtype);
#undef DD_FINISH_SIZED
#undef DD_FINISH
    return dd_check_launch("dd_retention_finish");
}
