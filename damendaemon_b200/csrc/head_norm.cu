// RMS norm over every head of the queries and keys, then the rotary rotation, in place and in one pass.
//
// A head x of head_dim values becomes x / sqrt(mean(x^2) + eps) * w, with one weight vector w [head_dim] for all
// query heads and another for all key heads (a null weight leaves that kind unnormed); then, if there are
// frequencies, the first 2 * n_pairs dimensions are rotated as in rotary.cu: pair i is (2i, 2i + 1) in the
// interleaved layout and (i, i + n_pairs) in the layout of halves, (a, b) -> (a c - b s, b c + a s) with the cosine
// and sine of position * f_i. The head is read once, kept as float32 in shared memory, and written once: the normed
// value is never rounded to the storage type before it is rotated. Sum of squares, root, angle, cosine and sine are
// float32 whatever the storage type.
//
// A block owns a token and a share of its heads: it computes the token's cosines and sines once (they serve every head),
// then each of its warps takes heads in turn. k may be null with k_heads == 0: a mixer that reads another layer's keys has
// queries only.
#include "common.cuh"

namespace {
constexpr int WARPS = 8;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
head_norm_rotary_kernel(T* __restrict__ q, T* __restrict__ k, int stride, const int* __restrict__ positions,
                        const float* __restrict__ freqs, const float* __restrict__ q_weight,
                        const float* __restrict__ k_weight, float eps, int q_heads, int k_heads, int head_dim,
                        int n_pairs, int interleaved, int heads_per_block) {
    extern __shared__ float staged[];             // [n_pairs] cosines, [n_pairs] sines, [WARPS][head_dim] a head per warp
    float* cosines = staged;
    float* sines = staged + n_pairs;
    dd_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const float p = (float)positions[t];          // positions are the step's input, not the projection's output
    for (int i = threadIdx.x; i < n_pairs; i += WARPS * 32) sincosf(p * freqs[i], &sines[i], &cosines[i]);
    __syncthreads();
    dd_grid_wait();
    float* x = staged + 2 * n_pairs + warp * head_dim;
    const int heads = q_heads + k_heads;
    const int h_end = min(heads, (int)(blockIdx.y + 1) * heads_per_block);
    for (int h = blockIdx.y * heads_per_block + warp; h < h_end; h += WARPS) {
        T* head = h < q_heads ? q + (size_t)t * stride + (size_t)h * head_dim : k + (size_t)t * stride + (size_t)(h - q_heads) * head_dim;
        const float* w = h < q_heads ? q_weight : k_weight;
        float sq = 0.f;
        for (int c = lane; c < head_dim; c += 32) {
            const float v = dd_to_f32(head[c]);
            x[c] = v;
            sq += v * v;
        }
        sq = dd_warp_sum(sq);
        if (w) {
            const float r = 1.0f / sqrtf(sq / (float)head_dim + eps);
            for (int c = lane; c < head_dim; c += 32) x[c] = x[c] * r * w[c];
        }
        __syncwarp();
        for (int i = lane; i < n_pairs; i += 32) {
            const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + n_pairs;
            const float cs = cosines[i], sn = sines[i];
            const float a = x[ia], b = x[ib];
            head[ia] = dd_from_f32<T>(a * cs - b * sn);
            head[ib] = dd_from_f32<T>(b * cs + a * sn);
        }
        if (w)
            for (int c = 2 * n_pairs + lane; c < head_dim; c += 32) head[c] = dd_from_f32<T>(x[c]);
        __syncwarp();                             // the next head of this warp overwrites x
    }
}

// 16 bytes of a head as float32 values, and back.
template <typename T> struct Piece;
template <> struct Piece<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
    __device__ static void store(float* p, const float* in) { *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]); }
};
template <> struct Piece<__nv_bfloat16> {
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
    __device__ static void store(__nv_bfloat16* p, const float* in) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&v);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// The layout of halves in 16-byte pieces: a head is shared by G neighbouring lanes (a power of two); lane j of them, if
// j < rotated, owns the piece j of the rotated stretch's first half and the piece j of its second half (their elements
// are each other's partners), else, if j < rotated + tail, the piece j - rotated of the dimensions behind the rotated
// stretch. The sum of squares goes over the G lanes in log2 G exchanges. A block owns a token: its cosines and sines are
// computed once; one pass of the block covers THREADS / G heads. About a thirteenth of the general kernel's instructions.
template <typename T, int G>
__global__ void __launch_bounds__(WARPS * 32)
head_norm_rotary_pieces_kernel(T* __restrict__ q, T* __restrict__ k, int stride, const int* __restrict__ positions,
                               const float* __restrict__ freqs, const float* __restrict__ q_weight,
                               const float* __restrict__ k_weight, float eps, int q_heads, int k_heads, int head_dim,
                               int n_pairs, int heads_per_block) {
    constexpr int V = Piece<T>::N;
    extern __shared__ __align__(16) float table[];       // [n_pairs] cosines, [n_pairs] sines
    float* cosines = table;
    float* sines = table + n_pairs;
    dd_launch_dependents();
    const int t = blockIdx.x;
    const float p = (float)positions[t];
    for (int i = threadIdx.x; i < n_pairs; i += WARPS * 32) sincosf(p * freqs[i], &sines[i], &cosines[i]);
    __syncthreads();
    dd_grid_wait();
    const int rotated = n_pairs / V, tail = (head_dim - 2 * n_pairs) / V;
    const int j = threadIdx.x % G;
    const int heads = q_heads + k_heads;
    const int h_first = blockIdx.y * heads_per_block, h_end = min(heads, h_first + heads_per_block);
    // every lane walks the same number of passes (the exchanges below take all 32 lanes); a lane without a head idles
    for (int h0 = h_first; h0 < h_end; h0 += WARPS * 32 / G) {
        const int h = h0 + threadIdx.x / G;
        const bool live = h < h_end && j < rotated + tail;
        T* head = nullptr;
        const float* w = nullptr;
        if (live) {
            head = h < q_heads ? q + (size_t)t * stride + (size_t)h * head_dim : k + (size_t)t * stride + (size_t)(h - q_heads) * head_dim;
            w = h < q_heads ? q_weight : k_weight;
        }
        const bool pair = j < rotated;
        const int at_a = pair ? j * V : 2 * n_pairs + (j - rotated) * V, at_b = n_pairs + j * V;
        float a[V], b[V];
#pragma unroll
        for (int i = 0; i < V; ++i) a[i] = b[i] = 0.f;
        if (live) {
            Piece<T>::load(head + at_a, a);
            if (pair) Piece<T>::load(head + at_b, b);
        }
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < V; ++i) sq = fmaf(a[i], a[i], fmaf(b[i], b[i], sq));
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (!live) continue;
        if (w) {
            const float r = 1.0f / sqrtf(sq / (float)head_dim + eps);
#pragma unroll
            for (int i = 0; i < V; i += 4) {
                const float4 wa = *reinterpret_cast<const float4*>(w + at_a + i);
                a[i] = a[i] * r * wa.x; a[i + 1] = a[i + 1] * r * wa.y; a[i + 2] = a[i + 2] * r * wa.z; a[i + 3] = a[i + 3] * r * wa.w;
                if (pair) {
                    const float4 wb = *reinterpret_cast<const float4*>(w + at_b + i);
                    b[i] = b[i] * r * wb.x; b[i + 1] = b[i + 1] * r * wb.y; b[i + 2] = b[i + 2] * r * wb.z; b[i + 3] = b[i + 3] * r * wb.w;
                }
            }
        }
        if (pair) {
            float ra[V], rb[V];
#pragma unroll
            for (int i = 0; i < V; ++i) {
                const float cs = cosines[j * V + i], sn = sines[j * V + i];
                ra[i] = a[i] * cs - b[i] * sn;
                rb[i] = b[i] * cs + a[i] * sn;
            }
            Piece<T>::store(head + at_a, ra);
            Piece<T>::store(head + at_b, rb);
        } else if (w) {
            Piece<T>::store(head + at_a, a);
        }
    }
}
}  // namespace

// q: [n_tokens] rows of `stride` elements with q_heads heads of head_dim; k likewise with k_heads heads (row views of
// one buffer; null with k_heads == 0). q_weight, k_weight: float32 [head_dim] or null. freqs: float32 [n_pairs] or
// null with n_pairs == 0 (norm only).
DD_API int dd_head_norm_rotary(void* q, void* k, int stride, const int* positions, const float* freqs, const float* q_weight,
                               const float* k_weight, float eps, int n_tokens, int q_heads, int k_heads, int head_dim,
                               int n_pairs, int interleaved, int dtype, void* stream) {
    if (n_tokens <= 0 || q_heads + k_heads <= 0) return 0;
    if (n_pairs < 0 || 2 * n_pairs > head_dim) return dd_fail("dd_head_norm_rotary: %d pairs do not fit a head of %d", n_pairs, head_dim);
    if (head_dim <= 0 || head_dim > 1024) return dd_fail("dd_head_norm_rotary: a head of %d is not supported (at most 1024)", head_dim);
    if ((k_heads > 0 && !k) || (q_heads > 0 && !q) || (n_pairs > 0 && !freqs))
        return dd_fail("dd_head_norm_rotary: a null pointer for heads or frequencies that are wanted");
    cudaStream_t s = (cudaStream_t)stream;
    // a token's heads are shared out over as many blocks as give the GPU two blocks an SM (at most a block per WARPS heads)
    const int heads = q_heads + k_heads;
    int groups = dd_ceil_div(296, n_tokens);
    if (groups > dd_ceil_div(heads, WARPS)) groups = dd_ceil_div(heads, WARPS);
    if (groups < 1) groups = 1;
    const int heads_per_block = dd_ceil_div(heads, groups);
    const dim3 grid(n_tokens, dd_ceil_div(heads, heads_per_block));
    // the layout of halves in whole 16-byte pieces: the kernel that moves pieces
    const int piece = dtype == DD_F32 ? 4 : 8;
    const int lanes = n_pairs / piece + (head_dim - 2 * n_pairs) / piece;        // lanes a head needs
    const bool aligned = !(((uintptr_t)q | (uintptr_t)k | (uintptr_t)q_weight | (uintptr_t)k_weight) & 15) && stride % piece == 0 &&
                         head_dim % piece == 0 && n_pairs % piece == 0;
    if (!interleaved && aligned && lanes >= 1 && lanes <= 32 && (dtype == DD_F32 || dtype == DD_BF16)) {
        int g = 1;
        while (g < lanes) g <<= 1;
        const size_t table_bytes = 2 * (size_t)n_pairs * sizeof(float);
#define DD_PIECES(T, G)                                                                                                     \
        dd_launch(head_norm_rotary_pieces_kernel<T, G>, grid, dim3(WARPS * 32), table_bytes, s, (T*)q, (T*)k, stride, positions, freqs, \
                  q_weight, k_weight, eps, q_heads, k_heads, head_dim, n_pairs, heads_per_block)
#define DD_PIECES_G(T)                                          \
        switch (g) {                                            \
            case 1: DD_PIECES(T, 1); break;                     \
            case 2: DD_PIECES(T, 2); break;                     \
            case 4: DD_PIECES(T, 4); break;                     \
            case 8: DD_PIECES(T, 8); break;                     \
            case 16: DD_PIECES(T, 16); break;                   \
            default: DD_PIECES(T, 32); break;                   \
        }
        if (dtype == DD_F32) { DD_PIECES_G(float) } else { DD_PIECES_G(__nv_bfloat16) }
#undef DD_PIECES_G
#undef DD_PIECES
        return dd_check_launch("dd_head_norm_rotary");
    }
    const size_t smem = ((size_t)WARPS * head_dim + 2 * (size_t)n_pairs) * sizeof(float);
    if (dtype == DD_F32)
        dd_launch(head_norm_rotary_kernel<float>, grid, dim3(WARPS * 32), smem, s, (float*)q, (float*)k, stride, positions,
                  freqs, q_weight, k_weight, eps, q_heads, k_heads, head_dim, n_pairs, interleaved, heads_per_block);
    else if (dtype == DD_BF16)
        dd_launch(head_norm_rotary_kernel<__nv_bfloat16>, grid, dim3(WARPS * 32), smem, s, (__nv_bfloat16*)q,
                  (__nv_bfloat16*)k, stride, positions, freqs, q_weight, k_weight, eps, q_heads, k_heads, head_dim,
                  n_pairs, interleaved, heads_per_block);
    else
        return dd_fail("dd_head_norm_rotary: unknown dtype %d", dtype);
    return dd_check_launch("dd_head_norm_rotary");
}
