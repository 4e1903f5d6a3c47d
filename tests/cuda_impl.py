"""The product's operators under the names ``cases.run_case`` uses; every
tensor argument is moved to the GPU and results come back to the host."""

import torch

import voyager_b200  # noqa: F401  (registers torch.ops.quantized_ops)

Q = torch.ops.quantized_ops
DEV = "cuda"


def _to_dev(a):
    if isinstance(a, torch.Tensor):
        return a.to(DEV)
    if isinstance(a, (list, tuple)) and a and isinstance(a[0], torch.Tensor):
        return type(a)(_to_dev(v) for v in a)
    return a


def _to_host(o):
    if isinstance(o, torch.Tensor):
        return o.cpu()
    if isinstance(o, (list, tuple)):
        return tuple(_to_host(v) for v in o)
    return o


def _wrap(fn):
    def call(*args, **kwargs):
        out = fn(*[_to_dev(a) for a in args], **{k: _to_dev(v) for k, v in kwargs.items()})
        torch.cuda.synchronize()
        return _to_host(out)

    return call


class CudaImpl:
    vmap = staticmethod(_wrap(Q.vmap))
    quantize = staticmethod(_wrap(Q.quantize))
    dequantize = staticmethod(_wrap(Q.dequantize))
    calculate_mx_qparam = staticmethod(_wrap(Q.calculate_mx_qparam))
    quantize_mx = staticmethod(_wrap(Q.quantize_mx))
    dequantize_mx = staticmethod(_wrap(Q.dequantize_mx))
    quantize_affine = staticmethod(_wrap(Q.quantize_affine))
    calculate_global_scale = staticmethod(_wrap(voyager_b200.calculate_global_scale))


CudaImpl.linear_mx = staticmethod(_wrap(Q.linear_mx))
CudaImpl.matmul_mx = staticmethod(_wrap(Q.matmul_mx))
CudaImpl.linear = staticmethod(_wrap(Q.linear))
CudaImpl.matmul = staticmethod(_wrap(Q.matmul))
CudaImpl.sdpa_mx = staticmethod(_wrap(Q.sdpa_mx))
CudaImpl.quantize_mx_transpose = staticmethod(_wrap(Q.quantize_mx_transpose))
CudaImpl.hadamard_rotate = staticmethod(_wrap(voyager_b200.ops.hadamard_rotate))
CudaImpl.hadamard_matrix = staticmethod(voyager_b200.ops.hadamard_matrix)

FQ = torch.ops.quantization
CudaImpl.fake_quant = staticmethod(_wrap(FQ.fake_quant))
CudaImpl.group_wise_affine_fake_quant = staticmethod(_wrap(FQ.group_wise_affine_fake_quant))
CudaImpl.mx_fake_quant = staticmethod(_wrap(FQ.mx_fake_quant))
CudaImpl.hadamard_amax = staticmethod(_wrap(FQ.hadamard_amax))


def _amax_observer(sequence, dtype, quant_max, history_len, ch_axis, power_2_scale):
    Q = voyager_b200.QScheme
    scheme = Q.PER_TENSOR_SYMMETRIC if ch_axis is None else Q.PER_CHANNEL_SYMMETRIC
    module = voyager_b200.observers.FusedAmaxObsFakeQuantize(dtype, scheme, quant_max, history_len, ch_axis,
                                                             power_2_scale, device=DEV)
    outs, scales = [], []
    for x in sequence.to(DEV):
        outs.append(module(x))
        scales.append(module.scale.clone())
    torch.cuda.synchronize()
    return torch.stack(outs).cpu(), torch.stack(scales).cpu()


CudaImpl.amax_observer = staticmethod(_amax_observer)

CudaImpl.filter_outlier = staticmethod(_wrap(Q.filter_outlier))
CudaImpl.quantize_mx_outlier = staticmethod(_wrap(Q.quantize_mx_outlier))
CudaImpl.slice_csr_tensor = staticmethod(_wrap(Q.slice_csr_tensor))
CudaImpl.spmm_csr = staticmethod(_wrap(Q.spmm_csr))
