"""The outlier side stream of ``quantized_ops`` on the CUDA kernels.

``filter_outlier``, ``quantize_mx_outlier``, ``slice_csr_tensor`` and ``spmm_csr`` (reference
``src/voyager_compiler/ops/quantized.py:1286-1644``, same schemas): elements whose magnitude
reaches a threshold leave the tensor as a CSR matrix of fixed capacity and are multiplied
separately in float32; ``linear_mx`` / ``matmul_mx`` add that product before their one rounding.

Unlike the reference, nothing here reads a value back to the host (no ``.item()``): counts
become row pointers by a device prefix sum and slices are gathers with device offsets, so the
operators can be captured in a CUDA graph.
"""

import math
from typing import Optional

import torch

from . import _native as N
from .ops import (_decode_and_scale, _dtype_id, _parse_layout, _stream, quantized_ops_lib)

Q = torch.ops.quantized_ops

quantized_ops_lib.define(
    "filter_outlier(Tensor input, float threshold, float max_pct=0.01) -> (Tensor, Tensor, Tensor, Tensor)")
quantized_ops_lib.define(
    "quantize_mx_outlier(Tensor self, Tensor qmap, SymInt[] axes, int block_size, float quant_max, "
    "bool force_scale_power_of_two=False, Tensor scale_qmap=None, Tensor output_code=None, float? threshold=None, "
    "float max_pct=0.01, SymInt indptr_offset=0) -> (Tensor, Tensor, Tensor, Tensor, Tensor)")
quantized_ops_lib.define(
    "slice_csr_tensor(Tensor data, Tensor indices, Tensor indptr, int dim=0, SymInt? start=None, SymInt? end=None, "
    "float size_factor=1.0) -> (Tensor, Tensor, Tensor)")
quantized_ops_lib.define(
    "spmm_csr(Tensor data, Tensor indices, Tensor indptr, Tensor B, Tensor? B_scale=None, Tensor? B_code=None, "
    'int? block_size=None, str weight_layout="kc", *, ScalarType? out_dtype=None) -> Tensor')


def _capacity(shape, max_pct: float) -> int:
    return int(math.prod(shape[-2:]) * max_pct)


def filter_outlier(input: torch.Tensor, threshold: float, max_pct: float = 0.01):
    """``(data, indices, indptr, inlier)``: the elements with ``|x| >= threshold`` as a CSR matrix per
    ``[rows, cols]`` matrix (``int(rows * cols * max_pct)`` entries, padded with 0 / -1, int32
    indices and row pointers) and the input with those elements zeroed (reference ``quantized.py:1323-1373``)."""
    x = input.contiguous()
    if x.dim() < 2:
        raise ValueError("filter_outlier takes matrices")
    rows, cols = x.shape[-2:]
    batch = x.shape[:-2]
    nb = int(math.prod(batch))
    cap = _capacity(x.shape, max_pct)
    thr = float(torch.tensor(threshold, dtype=x.dtype))        # the comparison happens in the tensor's dtype
    lib, dt, st = N.lib(), _dtype_id(x.dtype), _stream()
    counts = torch.empty(nb, rows, dtype=torch.int32, device=x.device)
    N.check(lib.vq_outlier_count(x.data_ptr(), dt, counts.data_ptr(), nb * rows, cols, thr, st), "vq_outlier_count")
    row_start = torch.zeros(nb, rows + 1, dtype=torch.int32, device=x.device)
    row_start[:, 1:] = counts.cumsum(1)
    data = torch.zeros(nb, cap, dtype=x.dtype, device=x.device)
    indices = torch.full((nb, cap), -1, dtype=torch.int32, device=x.device)
    inlier = torch.empty_like(x)
    N.check(lib.vq_outlier_fill(x.data_ptr(), dt, inlier.data_ptr(), data.data_ptr(), indices.data_ptr(),
                                row_start.data_ptr(), nb, rows, cols, thr, cap, st), "vq_outlier_fill")
    indptr = row_start.clamp_(max=cap)                           # an over-full matrix is truncated, as the hardware does
    return data.reshape(*batch, cap), indices.reshape(*batch, cap), indptr.reshape(*batch, rows + 1), inlier


def quantize_mx_outlier(input, qmap, axes, block_size, quant_max, force_scale_power_of_two=False, scale_qmap=None,
                        output_code=None, threshold=None, max_pct=0.01, indptr_offset=0):
    """``(data, indices, indptr, scale, inliers)``: outliers to a CSR, the rest through ``quantize_mx``
    (reference ``quantized.py:1405-1455``)."""
    data, indices, indptr, inliers = filter_outlier(input, threshold, max_pct)
    if indptr_offset:
        indptr = indptr + indptr_offset
    scale, inliers = Q.quantize_mx(inliers, qmap, axes, block_size, quant_max, force_scale_power_of_two, scale_qmap,
                                   output_code)
    return data, indices, indptr, scale, inliers


def _repad(values_at, count, cap, data, indices, column_shift=0):
    """First ``min(count, cap)`` entries taken from positions ``values_at`` (device indices)."""
    slot = torch.arange(cap, device=data.device)
    valid = slot < count
    src = values_at.clamp(0, max(data.shape[0] - 1, 0))
    new_data = torch.where(valid, data[src], torch.zeros((), dtype=data.dtype, device=data.device))
    new_indices = torch.where(valid, indices[src] - column_shift, torch.full((), -1, dtype=indices.dtype,
                                                                             device=data.device))
    return new_data, new_indices


def slice_csr_tensor(data, indices, indptr, dim=0, start=None, end=None, size_factor=1.0):
    """Rows (``dim`` 0) or columns (``dim`` 1) ``[start, end)`` of one CSR matrix, re-padded to
    ``int(len(data) * size_factor)`` entries (reference ``quantized.py:1500-1541``)."""
    dim = dim + 2 if dim < 0 else dim
    if dim not in (0, 1):
        raise ValueError(f"Cannot slice sparse CSR matrix along dim {dim}")
    cap = int(data.shape[0] * size_factor)
    if data.shape[0] == 0:
        return data.new_zeros(cap), indices.new_full((cap,), -1), (indptr[start:end + 1] * 0 if dim == 0 else indptr * 0)
    slot = torch.arange(cap, device=data.device)
    if dim == 0:
        first = indptr[start].to(torch.int64)
        new_indptr = (indptr[start:end + 1] - indptr[start]).clamp(max=cap)
        count = indptr[end].to(torch.int64) - first
        new_data, new_indices = _repad(first + slot, count, cap, data, indices)
        return new_data, new_indices, new_indptr
    nse = indptr[-1].to(torch.int64)
    position = torch.arange(data.shape[0], device=data.device)
    keep = (indices >= start) & (indices < end) & (position < nse)
    kept_before = torch.cat([keep.new_zeros(1, dtype=torch.int64), keep.to(torch.int64).cumsum(0)])
    new_indptr = kept_before[indptr.to(torch.int64).clamp(0, data.shape[0])].to(indptr.dtype).clamp(max=cap)
    # compact: entry i goes to slot kept_before[i] when kept and inside the capacity, else to a spare slot
    target = torch.where(keep & (kept_before[:-1] < cap), kept_before[:-1], torch.full_like(position, cap))
    new_data = data.new_zeros(cap + 1).scatter_(0, target, data)[:cap]
    new_indices = indices.new_full((cap + 1,), -1).scatter_(0, target, indices - start)[:cap]
    filled = slot < kept_before[-1]
    new_data = torch.where(filled, new_data, torch.zeros((), dtype=data.dtype, device=data.device))
    new_indices = torch.where(filled, new_indices, torch.full((), -1, dtype=indices.dtype, device=data.device))
    return new_data, new_indices, new_indptr


def spmm_csr(data, indices, indptr, B, B_scale=None, B_code=None, block_size=None, weight_layout="kc", *,
             out_dtype: Optional[torch.dtype] = None):
    """CSR x dense, summed in float32 and rounded to ``out_dtype`` (or ``B``'s dtype); ``B`` is read back
    through its codebook and block scales first and is ``[out, contraction]`` for ``"kc"``
    (reference ``quantized.py:1574-1644``)."""
    if weight_layout not in ("kc", "ck"):
        raise ValueError(weight_layout)
    if B_code is not None or B_scale is not None:
        B = _decode_and_scale(B, B_scale, B_code, block_size)
    B = B.contiguous()
    batch = indptr.shape[:-1]
    nb = int(math.prod(batch))
    rows = indptr.shape[-1] - 1
    cap = data.shape[-1]
    if weight_layout == "kc":
        n_out, k = B.shape[-2], B.shape[-1]
        ld_k, ld_n = 1, k
    else:
        k, n_out = B.shape[-2], B.shape[-1]
        ld_k, ld_n = n_out, 1
    stride_b = B.shape[-2] * B.shape[-1] if B.dim() > 2 else 0
    dtype = B.dtype if out_dtype is None else out_dtype
    out = torch.empty(nb, rows, n_out, dtype=dtype, device=B.device)
    data2 = data.reshape(nb, cap).contiguous()
    indices2 = indices.reshape(nb, cap).to(torch.int32).contiguous()
    indptr2 = indptr.reshape(nb, rows + 1).to(torch.int32).contiguous()
    N.check(N.lib().vq_spmm_csr(data2.data_ptr(), _dtype_id(data2.dtype), indices2.data_ptr(), indptr2.data_ptr(),
                                B.data_ptr(), _dtype_id(B.dtype), out.data_ptr(), _dtype_id(dtype), nb, rows, n_out, k,
                                cap, stride_b, ld_k, ld_n, _stream()), "vq_spmm_csr")
    return out.reshape(*batch, rows, n_out)


quantized_ops_lib.impl("filter_outlier", N.device_guarded(filter_outlier), "CUDA")
quantized_ops_lib.impl("quantize_mx_outlier", N.device_guarded(quantize_mx_outlier), "CUDA")
quantized_ops_lib.impl("slice_csr_tensor", N.device_guarded(slice_csr_tensor), "CUDA")
quantized_ops_lib.impl("spmm_csr", N.device_guarded(spmm_csr), "CUDA")


@torch.library.register_fake("quantized_ops::filter_outlier")
def _(input, threshold, max_pct=0.01):
    batch, (rows, _) = input.shape[:-2], input.shape[-2:]
    cap = _capacity(input.shape, max_pct)
    return (input.new_empty((*batch, cap)), input.new_empty((*batch, cap), dtype=torch.int32),
            input.new_empty((*batch, rows + 1), dtype=torch.int32), torch.empty_like(input))


@torch.library.register_fake("quantized_ops::quantize_mx_outlier")
def _(input, qmap, axes, block_size, quant_max, force_scale_power_of_two=False, scale_qmap=None, output_code=None,
      threshold=None, max_pct=0.01, indptr_offset=0):
    batch, (rows, _) = input.shape[:-2], input.shape[-2:]
    cap = _capacity(input.shape, max_pct)
    scale_shape = list(input.shape)
    for axis in axes:
        scale_shape[axis] = math.ceil(scale_shape[axis] / block_size)
    return (input.new_empty((*batch, cap)), input.new_empty((*batch, cap), dtype=torch.int32),
            input.new_empty((*batch, rows + 1), dtype=torch.int32), input.new_empty(scale_shape),
            torch.empty_like(input, memory_format=torch.contiguous_format))


@torch.library.register_fake("quantized_ops::slice_csr_tensor")
def _(data, indices, indptr, dim=0, start=None, end=None, size_factor=1.0):
    cap = int(data.shape[0] * size_factor)
    new_indptr = indptr[start:end + 1] if dim in (0, -2) else indptr
    return data.new_empty(cap), indices.new_empty(cap), torch.empty_like(new_indptr)


@torch.library.register_fake("quantized_ops::spmm_csr")
def _(data, indices, indptr, B, B_scale=None, B_code=None, block_size=None, weight_layout="kc", *, out_dtype=None):
    n_out = B.shape[-2] if weight_layout == "kc" else B.shape[-1]
    return B.new_empty((*indptr.shape[:-1], indptr.shape[-1] - 1, n_out), dtype=out_dtype or B.dtype)
