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
