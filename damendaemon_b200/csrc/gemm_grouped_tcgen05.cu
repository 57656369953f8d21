// Grouped bfloat16 product on the 5th-generation tensor cores: rows of X that come in tiles, each tile multiplied
// with the matrix of its own group (an expert) out of a stack W[groups][N, K]:
//
//     out[r, n] = sum_k X[r, k] * W[group(tile of r)][n, k]
//
// and, fused (DUAL), the gated unit of two such products over the same rows: the stack holds 2N rows per group, N
// gate rows followed by N up rows, and out[r, n] = g * sigmoid(alpha g) * (u + 1) with g = min(gate, limit),
// u = clamp(up, -limit, limit), or another form of the unit (dd_gated_value in common.cuh: silu(gate) * up, tanh-gelu(gate)
// * up), computed in float32 from the two accumulators.
//
// The product is computed transposed, D^T = W . X^T: 128 weight rows are the lanes of the accumulator and a tile's
// T rows of X (16, 32, 64 or 128) its columns, so that a step in which an expert gets a few tokens wastes no
// tensor-core rows and still streams the expert's matrix from 128-row blocks spread over the SMs. A block owns one
// (128 features, row tile) pair: one thread feeds TMA (64-element k slices with the 128-byte swizzle into a ring of
// stages), one issues tcgen05.mma into tensor memory (DUAL: two accumulators side by side that share the X tile, so
// gate and up of a feature meet in one thread's registers), four warps read the accumulators back and store. A tile
// whose group is negative holds no rows: its blocks leave at once. The group of a tile is only known on the device
// (after the kernel that sorted the rows), so nothing is fetched before the wait for the kernel before.
//
// Every mbarrier wait is bounded (tcgen05.cuh): on a timeout bit 8 of the error word is set and the block leaves.
#include "common.cuh"
#include "tcgen05.cuh"

namespace {
constexpr int BM = 128, BK = 64, UMMA_K = 16, THREADS = 192;

struct GroupedParams {
    const int* tile_group;       // [row tiles]: the group of a tile, negative for a tile without rows
    void* out;                   // [rows, ldo] bf16 or f32
    int* error_flag;
    int ldo, out_dtype;
    int N, K;                    // output features per group, reduction
    int rows_per_group;          // rows of W per group: N, or 2N with the gated unit
    float limit, alpha;
    int form;                    // DD_GATED_*: which gated unit
};

template <int T, bool DUAL> struct GroupedConfig {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int W_BYTES = DUAL ? 2 * A_BYTES : A_BYTES;
    static constexpr int X_BYTES = T * BK * 2;
    static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
    // Two blocks share an SM (110 KB of stages each; their accumulators fit tensor memory side by side): a block owns
    // one tile, so the loads of one run under the products of the other and one's epilogue under the other's products.
    static constexpr int FIT = 110 * 1024 / STAGE_BYTES;
    static constexpr int STAGES = FIT < 8 ? FIT : 8;
    static constexpr int WANTED = DUAL ? 2 * T : T;
    static constexpr int TMEM_COLS = WANTED < 32 ? 32 : WANTED;          // T is a power of two: so is this
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <int T, bool DUAL>
__global__ void __launch_bounds__(THREADS, 2)
gemm_grouped_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const GroupedParams p) {
    using C = GroupedConfig<T, DUAL>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + C::STAGES;
    uint64_t* acc_bar = empty_bar + C::STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            tc::mbar_init(&full_bar[s], 1);
            tc::mbar_init(&empty_bar[s], 1);
        }
        tc::mbar_init(acc_bar, 1);
        *abort_flag = 0;
        tc::fence_barrier_init();
        tc::fence_proxy_async();
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, C::TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    dd_launch_dependents();
    dd_grid_wait();              // the tile's group and the rows are earlier kernels' results

    const int n0 = blockIdx.x * BM, row0 = blockIdx.y * T;
    const int group = p.tile_group[blockIdx.y];
    const int kblocks = (p.K + BK - 1) / BK;
    if (group >= 0) {
        if (warp == 0) {
            if (tc::elect_one()) {
                tc::prefetch_tensormap(&map_w);
                tc::prefetch_tensormap(&map_x);
                const int w_row = group * p.rows_per_group + n0;
                for (int i = 0; i < kblocks; ++i) {
                    const int s = i % C::STAGES;
                    const uint32_t phase = (i / C::STAGES) & 1;
                    if (!tc::mbar_wait(&empty_bar[s], phase ^ 1, abort_flag)) break;
                    uint8_t* stage = tiles + s * C::STAGE_BYTES;
                    tc::mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
                    tc::tma_load_2d(stage, &map_w, i * BK, w_row, &full_bar[s]);
                    if (DUAL) tc::tma_load_2d(stage + C::A_BYTES, &map_w, i * BK, w_row + p.N, &full_bar[s]);
                    tc::tma_load_2d(stage + C::W_BYTES, &map_x, i * BK, row0, &full_bar[s]);
                }
            }
        } else if (warp == 1) {
            if (tc::elect_one()) {
                constexpr uint32_t idesc = tc::idesc_bf16_f32(BM, T);
                bool ok = true;
                for (int i = 0; i < kblocks; ++i) {
                    const int s = i % C::STAGES;
                    const uint32_t phase = (i / C::STAGES) & 1;
                    if (!tc::mbar_wait(&full_bar[s], phase, abort_flag)) { ok = false; break; }
                    tc::fence_after_sync();
                    const uint32_t a_addr = tc::smem_u32(tiles + s * C::STAGE_BYTES);
                    const uint32_t x_addr = a_addr + C::W_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t dx = tc::smem_desc_sw128(x_addr + k * UMMA_K * 2);
                        tc::mma_bf16(tmem_base, tc::smem_desc_sw128(a_addr + k * UMMA_K * 2), dx, idesc, (i > 0 || k > 0) ? 1u : 0u);
                        if (DUAL)
                            tc::mma_bf16(tmem_base + T, tc::smem_desc_sw128(a_addr + C::A_BYTES + k * UMMA_K * 2), dx, idesc,
                                         (i > 0 || k > 0) ? 1u : 0u);
                    }
                    tc::mma_commit(&empty_bar[s]);        // the stage is free once these MMAs have read it
                }
                if (ok) tc::mma_commit(acc_bar);          // the accumulators are complete
            }
        } else {
            // epilogue: warp w may touch TMEM lanes 32 * (w % 4) .. + 31; a thread owns output feature n
            const int quarter = warp & 3;
            const int n = n0 + quarter * 32 + lane;
            if (tc::mbar_wait(acc_bar, 0, abort_flag)) {
                tc::fence_after_sync();
                const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
                for (int c0 = 0; c0 < T; c0 += 16) {
                    uint32_t g[16], u[16];
                    tc::tmem_ld_x16(lane_addr + c0, g);
                    if (DUAL) tc::tmem_ld_x16(lane_addr + T + c0, u);
                    tc::tmem_ld_wait();
                    if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            float v = __uint_as_float(g[j]);
                            if (DUAL) v = dd_gated_value<true>(v, __uint_as_float(u[j]), p.form, p.limit, p.alpha);
                            const size_t at = (size_t)(row0 + c0 + j) * p.ldo + n;
                            if (p.out_dtype == DD_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(v);
                            else reinterpret_cast<float*>(p.out)[at] = v;
                        }
                    }
                }
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicOr(p.error_flag, 8);
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// rows x K bf16 matrix with row stride ld elements; boxes of box_rows x 64, 128-byte swizzle; beyond the matrix: zeros
int grouped_map(CUtensorMap* map, const void* base, long long rows, int K, int ld, int box_rows, const char* what) {
    static EncodeTiled enc = nullptr;
    if (!enc) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            enc = reinterpret_cast<EncodeTiled>(sym);
    }
    if (!enc) return dd_fail("dd_gemm_grouped_tcgen05: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return dd_fail("dd_gemm_grouped_tcgen05: cannot describe %s to TMA (driver error %d)", what, (int)r);
    return 0;
}

template <int T, bool DUAL>
int launch_grouped(const CUtensorMap& mw, const CUtensorMap& mx, const GroupedParams& p, int row_tiles, cudaStream_t s) {
    using C = GroupedConfig<T, DUAL>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_grouped_kernel<T, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return dd_fail("dd_gemm_grouped_tcgen05: shared memory of %d bytes refused: %s", C::SMEM_BYTES, cudaGetErrorString(e));
        configured = true;
    }
    dd_launch(gemm_grouped_kernel<T, DUAL>, dim3(dd_ceil_div(p.N, BM), row_tiles), dim3(THREADS), (size_t)C::SMEM_BYTES, s, mw, mx, p);
    return dd_check_launch("dd_gemm_grouped_tcgen05");
}
}  // namespace

// X [rows, K] bf16 (row stride ldx) in tiles of `tile` rows (16, 32, 64 or 128; rows a multiple of it); W: a stack of
// `groups` matrices of rows_per_group rows of K (row stride ldw, the matrices one after the other); tile_group: device
// array [rows / tile]. dual == 0: rows_per_group == N, out = X . W[g]^T. dual != 0: rows_per_group == 2 N (gate rows, up
// rows), out = gated unit (form: DD_GATED_*) of the two products with `limit` and `alpha`. out: [rows, N] bf16 or f32, row stride ldo.
DD_API int dd_gemm_grouped_tcgen05(const void* X, int ldx, const void* W, int ldw, int groups, int rows_per_group,
                                   const int* tile_group, void* out, int ldo, int rows, int N, int K, int tile, int dual,
                                   float limit, float alpha, int out_dtype, int* error_flag, void* stream, int form) {
    if (rows <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ldx % 8 || ldw % 8)
        return dd_fail("dd_gemm_grouped_tcgen05: K=%d and the row strides (%d, %d) must be multiples of 8 (TMA needs 16-byte rows)", K, ldx, ldw);
    if (((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return dd_fail("dd_gemm_grouped_tcgen05: operands must be 16-byte aligned");
    if (out_dtype != DD_BF16 && out_dtype != DD_F32) return dd_fail("dd_gemm_grouped_tcgen05: unknown output dtype %d", out_dtype);
    if (rows % tile || rows / tile > 65535) return dd_fail("dd_gemm_grouped_tcgen05: %d rows are not tiles of %d (at most 65535)", rows, tile);
    if (groups <= 0 || rows_per_group != (dual ? 2 * N : N) || !tile_group)
        return dd_fail("dd_gemm_grouped_tcgen05: %d rows per group do not fit N=%d", rows_per_group, N);
    GroupedParams p;
    p.tile_group = tile_group; p.out = out; p.error_flag = error_flag; p.ldo = ldo; p.out_dtype = out_dtype; p.N = N; p.K = K;
    p.rows_per_group = rows_per_group; p.limit = limit; p.alpha = alpha; p.form = form;
    CUtensorMap mw, mx;
    if (int e = grouped_map(&mw, W, (long long)groups * rows_per_group, K, ldw, BM, "the stacked matrices")) return e;
    if (int e = grouped_map(&mx, X, rows, K, ldx, tile, "the rows")) return e;
    cudaStream_t s = (cudaStream_t)stream;
    const int row_tiles = rows / tile;
#define DD_GROUPED(T)                                                                      \
    case T: return dual ? launch_grouped<T, true>(mw, mx, p, row_tiles, s) : launch_grouped<T, false>(mw, mx, p, row_tiles, s);
    switch (tile) {
        DD_GROUPED(16)
        DD_GROUPED(32)
        DD_GROUPED(64)
        DD_GROUPED(128)
    }
#undef DD_GROUPED
    return dd_fail("dd_gemm_grouped_tcgen05: tile %d is not one of 16, 32, 64, 128", tile);
}
