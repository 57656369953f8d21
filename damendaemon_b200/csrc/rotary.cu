// Rotary position encoding of queries and keys, in place, before they are cached and attended.
//
// The first 2 * n_pairs dimensions of every head are rotated, the rest pass unchanged. Pair i of a head is
// (2i, 2i + 1) in the interleaved layout and (i, i + n_pairs) in the layout of halves. At position p the pair (a, b)
// becomes (a c - b s, b c + a s) with c = magnitude * cos(p f_i), s = magnitude * sin(p f_i). The frequencies f_i
// are a float32 table of the caller's (plain, or blended for a longer context), so any scaling rule is the host's.
// Position, angle, cosine, sine and the rotation are float32 whatever the storage type; sincosf is the
// exact function (an angle reaches thousands of radians).
#include "common.cuh"

namespace {
constexpr int THREADS = 256, PER = 4;      // pairs a thread has in flight at once

// A pair of neighbours is one aligned 4- or 8-byte word: one access instead of two.
template <typename T> struct Pair;
template <> struct Pair<float> {
    __device__ static void load(const float* p, float& a, float& b) { const float2 v = *reinterpret_cast<const float2*>(p); a = v.x; b = v.y; }
    __device__ static void store(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};
template <> struct Pair<__nv_bfloat16> {
    __device__ static void load(const __nv_bfloat16* p, float& a, float& b) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
        a = __uint_as_float(w << 16);
        b = __uint_as_float(w & 0xffff0000u);
    }
    __device__ static void store(__nv_bfloat16* p, float a, float b) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        *reinterpret_cast<uint32_t*>(p) = *reinterpret_cast<const uint32_t*>(&v);
    }
};

// WORDS: neighbours are paired and every pair is an aligned word (decided by the launcher), so no branch stands
// between the loads of a pass.
template <typename T, bool WORDS>
__global__ void __launch_bounds__(THREADS)
rotary_kernel(T* __restrict__ q, T* __restrict__ k, int stride, const int* __restrict__ positions,
              const float* __restrict__ freqs, float magnitude, int q_heads, int k_heads, int head_dim, int n_pairs,
              int interleaved) {
    extern __shared__ float cs[];                 // [n_pairs] cosines, [n_pairs] sines of this token
    dd_launch_dependents();
    const int t = blockIdx.x;
    const float p = (float)positions[t];          // positions are the step's input, not the projection's output
    for (int i = threadIdx.x; i < n_pairs; i += THREADS) {
        float sn, c;
        sincosf(p * freqs[i], &sn, &c);
        cs[i] = c * magnitude;
        cs[n_pairs + i] = sn * magnitude;
    }
    __syncthreads();
    dd_grid_wait();
    const int items = (q_heads + k_heads) * n_pairs;
    T* q_row = q + (size_t)t * stride;
    T* k_row = k + (size_t)t * stride;
    // A thread reads PER pairs, then rotates and writes them: the loads of a pass are in flight together (one pair
    // at a time, each pass of the loop cost a trip to memory: 5.8 us for eight tokens).
    for (int base = 0; base < items; base += THREADS * PER) {
        float a[PER], b[PER];
        T* at[PER];
        int pair[PER];
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            const int item = base + u * THREADS + threadIdx.x;
            const bool live = item < items;
            const int h = live ? item / n_pairs : 0;
            pair[u] = live ? item - h * n_pairs : -1;
            T* head = h < q_heads ? q_row + (size_t)h * head_dim : k_row + (size_t)(h - q_heads) * head_dim;
            at[u] = head + (interleaved ? 2 * max(pair[u], 0) : max(pair[u], 0));
            a[u] = b[u] = 0.f;
            if (WORDS) {
                if (live) Pair<T>::load(at[u], a[u], b[u]);
            } else if (live) {
                a[u] = dd_to_f32(at[u][0]);
                b[u] = dd_to_f32(at[u][interleaved ? 1 : n_pairs]);
            }
        }
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            if (pair[u] < 0) continue;
            const float c = cs[pair[u]], sn = cs[n_pairs + pair[u]];
            if (WORDS) {
                Pair<T>::store(at[u], a[u] * c - b[u] * sn, b[u] * c + a[u] * sn);
                continue;
            }
            at[u][0] = dd_from_f32<T>(a[u] * c - b[u] * sn);
            at[u][interleaved ? 1 : n_pairs] = dd_from_f32<T>(b[u] * c + a[u] * sn);
        }
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
    if (dtype != DD_F32 && dtype != DD_BF16) return dd_fail("dd_rotary: unknown dtype %d", dtype);
    // neighbours as one word: when every pair starts on an even element of a row that starts on a whole word
    const size_t word = dtype == DD_F32 ? 8 : 4;
    const bool words = interleaved && !(stride & 1) && !(head_dim & 1) && !(((uintptr_t)q | (uintptr_t)k) & (word - 1));
#define DD_ROTARY(T, W)                                                                                                  \
    dd_launch(rotary_kernel<T, W>, dim3(n_tokens), dim3(THREADS), smem, s, (T*)q, (T*)k, stride, positions, freqs, magnitude, \
              q_heads, k_heads, head_dim, n_pairs, interleaved)
    if (dtype == DD_F32) {
        if (words) DD_ROTARY(float, true);
        else DD_ROTARY(float, false);
    } else {
        if (words) DD_ROTARY(__nv_bfloat16, true);
        else DD_ROTARY(__nv_bfloat16, false);
    }
#undef DD_ROTARY
    return dd_check_launch("dd_rotary");
}
