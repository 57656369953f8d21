"""Matrix products of the parts: one call that picks the kernel for the engine dtype."""
from __future__ import annotations

import torch

from .. import kernels


def linear(runtime, a, w, bias=None, residual=None, activation=None, out_dtype=None, out=None):
    """act(a @ w.T + bias) (+ residual). float32 engine: CUDA-core float32 kernel.
    bfloat16 engine: the tcgen05 tensor-core kernel, unless the runtime asks for 'simt' or the
    reduction width is no multiple of 8 (then the CUDA-core kernel with bfloat16 operands)."""
    if a.dtype == torch.float32 or runtime.gemm == "simt":
        return kernels.gemm_simt(a, w, bias, residual, activation, out_dtype, out)
    if a.shape[1] % 8 or a.stride(0) % 8 or w.stride(0) % 8:
        # TMA wants 16-byte rows; a reduction width that is no multiple of 8 runs on the CUDA cores instead
        return kernels.gemm_simt(a, w, bias, residual, activation, out_dtype or torch.bfloat16, out)
    return kernels.gemm_tcgen05(a, w, bias, residual, activation, out_dtype, out)


def grouped_on_tensor_cores(runtime, dtype, *reductions):
    """Whether grouped products over these reduction widths run on the tensor cores: bfloat16, and every width a
    multiple of 8 (TMA needs 16-byte rows). One answer for all products of a part: they share the rows' tiles."""
    return dtype == torch.bfloat16 and runtime.gemm != "simt" and all(k % 8 == 0 for k in reductions)


def grouped_tile(tensor_cores, pairs, groups):
    """Rows per tile of the grouped products: every group's rows start on a multiple of it. The tensor-core kernel
    takes 16 to 128: about twice the rows a group gets on average, so that few tiles are mostly padding and few groups
    need several. The CUDA-core kernel has one tile size."""
    if not tensor_cores:
        return kernels.simt_group_tile()
    want = 2 * pairs // max(1, groups)
    return next((t for t in kernels.GROUPED_TCGEN05_TILES if t >= want), kernels.GROUPED_TCGEN05_TILES[-1])


def grouped_linear(tensor_cores, a, w, tile_group, tile, out_dtype=None):
    """Rows of a in tiles of ``tile``; tile i is multiplied with w[tile_group[i]] (w: [groups, out, in]); tiles whose
    group is negative are skipped."""
    if tensor_cores:
        return kernels.gemm_grouped_tcgen05(a, w, tile_group, tile, out_dtype=out_dtype or a.dtype)
    return kernels.gemm_simt_grouped(a, w, tile_group, out_dtype=out_dtype or a.dtype)


def grouped_gated_unit(tensor_cores, a, gate_up, tile_group, tile, limit, alpha, form="clamped_swish"):
    """The gated unit (form: one of kernels.GATED_FORMS) over grouped rows: gate_up [groups, 2 * inner, in] holds a group's
    gate rows, then its up rows. On the tensor cores both products and the unit are one kernel; else a grouped product and
    the unit's own kernel."""
    if tensor_cores:
        return kernels.gemm_grouped_tcgen05(a, gate_up, tile_group, tile, gated=(limit, alpha, form))
    return kernels.gated_unit(kernels.gemm_simt_grouped(a, gate_up, tile_group), limit, alpha, form=form)
