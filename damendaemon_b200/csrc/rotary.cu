// Rotary position encoding of queries and keys, in place, before they are cached and attended.
//
// The first 2 * n_pairs dimensions of every head are rotated, the rest pass unchanged. Pair i of a head is
// (2i, 2i + 1) in the interleaved layout and (i, i + n_pairs) in the layout of halves. At position p the pair (a, b)
// becomes (a c - b s, b c + a s) with c = magnitude * cos(p f_i), s = magnitude * sin(p f_i). The frequencies f_i
// are a float32 table of the caller's (plain, or blended for a longer context), so any scaling rule is the host's.
// Position, angle, cosine, sine and the rotation are float32 whatever the storage type; cosf and sinf are the
// exact functions (an angle reaches thousands of radians).
#include "common.cuh"

namespace {
template <typename T>
__global__ void __launch_bounds__(128)
rotary_kernel(T* __restrict__ q, T* __restrict__ k, int stride, const int* __restrict__ positions,
              const float* __restrict__ freqs, float magnitude, int q_heads, int k_heads, int head_dim, int n_pairs,
              int interleaved) {
    extern __shared__ float cs[];                 // [n_pairs] cosines, [n_pairs] sines of this token
    dd_launch_dependents();
    const int t = blockIdx.x;
    const float p = (float)positions[t];          // positions are the step's input, not the projection's output
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const float a = p * freqs[i];
        cs[i] = cosf(a) * magnitude;
        cs[n_pairs + i] = sinf(a) * magnitude;
    }
    __syncthreads();
    dd_grid_wait();
    const int items = (q_heads + k_heads) * n_pairs;
    for (int item = threadIdx.x; item < items; item += blockDim.x) {
        const int h = item / n_pairs, i = item - h * n_pairs;
        T* row = h < q_heads ? q + (size_t)t * stride + (size_t)h * head_dim
                             : k + (size_t)t * stride + (size_t)(h - q_heads) * head_dim;
        const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + n_pairs;
        const float a = dd_to_f32(row[ia]), b = dd_to_f32(row[ib]);
        const float c = cs[i], s = cs[n_pairs + i];
        row[ia] = dd_from_f32<T>(a * c - b * s);
        row[ib] = dd_from_f32<T>(b * c + a * s);
    }
}
}  // namespace

// q: [n_tokens] rows of `stride` elements with q_heads heads of head_dim; k likewise with k_heads heads (row views
// of one buffer, what a fused projection leaves). freqs: float32 [n_pairs] on the device.
DD_API int dd_rotary(void* q, void* k, int stride, const int* positions, const float* freqs, float magnitude,
                     int n_tokens, int q_heads, int k_heads, int head_dim, int n_pairs, int interleaved, int dtype,
                     void* stream) {
    if (n_tokens <= 0 || n_pairs <= 0) return 0;
    if (2 * n_pairs > head_dim) return dd_fail("dd_rotary: %d pairs do not fit a head of %d", n_pairs, head_dim);
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = 2 * (size_t)n_pairs * sizeof(float);
    if (dtype == DD_F32)
        dd_launch(rotary_kernel<float>, dim3(n_tokens), dim3(128), smem, s, (float*)q, (float*)k, stride, positions, freqs,
                  magnitude, q_heads, k_heads, head_dim, n_pairs, interleaved);
    else if (dtype == DD_BF16)
        dd_launch(rotary_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), smem, s, (__nv_bfloat16*)q, (__nv_bfloat16*)k,
                  stride, positions, freqs, magnitude, q_heads, k_heads, head_dim, n_pairs, interleaved);
    else
        return dd_fail("dd_rotary: unknown dtype %d", dtype);
    return dd_check_launch("dd_rotary");
}
