"""Delayed-scaling fake-quantizer for the per-tensor and per-channel schemes, state on the device.

The counterpart of the reference's ``FusedAmaxObsFakeQuantize``
(``src/voyager_compiler/quantization/fake_quantize.py:330-447``): same class name, constructor
arguments, switches and ``scale`` / ``qmap`` / ``amax_history`` buffers, so code that builds
observers from a spec string finds the same interface.  What it computes: the module remembers
the absolute maxima of the last ``amax_history_len`` tensors it saw (one per tensor, or one per
channel along ``ch_axis``) and scales by the largest of them; a tensor is quantized with the
scale of its predecessors, before its own maximum counts, so the first call uses scale 1.

How it is kept here: ``amax_history`` is a ring ``[length, channels]`` with a device-side write
position per channel, and one small kernel (``vq_amax_history_update``) takes the ring's
maximum, derives the scale and stores the new amax.  A forward is three launches -- the tensor's
amax (``vq_amax``), the ring update, the fake-quantize -- with no host read, so it can sit
inside a captured CUDA graph.  (The reference rolls the whole history tensor every call; only the
order of the rows differs, the set of remembered maxima and therefore every scale is the same.)
"""

from typing import Optional

import torch

from . import _native as N
from .formats import QScheme, get_quantization_map
from .ops import _dtype_id, _stream, tensor_amax


class FusedAmaxObsFakeQuantize(torch.nn.Module):
    def __init__(self, dtype: str, qscheme: QScheme, quant_max: float, amax_history_len: int,
                 ch_axis: Optional[int] = None, power_2_scale: bool = False, device=None, **unused) -> None:
        if qscheme not in (QScheme.PER_TENSOR_SYMMETRIC, QScheme.PER_CHANNEL_SYMMETRIC):
            raise ValueError(f"{qscheme} is not a per-tensor or per-channel scheme")
        if amax_history_len < 1:
            raise ValueError("amax_history_len must be at least 1")
        super().__init__()
        self.dtype = dtype
        self.qscheme, self.quant_max = qscheme, quant_max
        self.amax_history_len, self.ch_axis, self.power_2_scale = amax_history_len, ch_axis, power_2_scale
        self.is_per_channel = qscheme == QScheme.PER_CHANNEL_SYMMETRIC
        self.register_buffer("qmap", get_quantization_map(dtype, device), persistent=False)
        self.register_buffer("scale", torch.tensor([1.0], dtype=torch.float, device=device))
        self.register_buffer("amax_history", torch.tensor([], dtype=torch.float, device=device))
        self.register_buffer("ring_position", torch.zeros(0, dtype=torch.int32, device=device), persistent=False)
        self.register_buffer("fake_quant_enabled", torch.tensor([1], dtype=torch.uint8))
        self.register_buffer("observer_enabled", torch.tensor([1], dtype=torch.uint8))
        # host copies of the two switches: forward never reads a device value
        self._observe, self._quantize = True, True

    def enable_observer(self, enabled: bool = True) -> None:
        self._observe = enabled
        self.observer_enabled[0] = int(enabled)

    def disable_observer(self) -> None:
        self.enable_observer(False)

    def enable_fake_quant(self, enabled: bool = True) -> None:
        self._quantize = enabled
        self.fake_quant_enabled[0] = int(enabled)

    def disable_fake_quant(self) -> None:
        self.enable_fake_quant(False)

    def _allocate(self, amax_shape, dtype, device) -> None:
        """Empty ring, write positions at 0 and scale 1, shaped for the first tensor seen."""
        self.amax_history = torch.zeros((self.amax_history_len, *amax_shape), dtype=dtype, device=device)
        self.scale = torch.ones(tuple(amax_shape), dtype=dtype, device=device)
        self.ring_position = torch.zeros(max(self.scale.numel(), 1), dtype=torch.int32, device=device)

    def _tensor_amax(self, x: torch.Tensor) -> torch.Tensor:
        if not self.is_per_channel:
            return tensor_amax(x)                                   # 0-d float32, one pass, no |x| temporary
        axis = self.ch_axis % x.ndim
        return x.abs().amax(dim=[i for i in range(x.ndim) if i != axis], keepdim=True)

    @torch.no_grad()
    def observe(self, x: torch.Tensor) -> None:
        """Derive ``scale`` from the maxima remembered so far, then remember ``x``'s."""
        if not x.is_cuda:
            raise NotImplementedError("the delayed-scaling observer runs on CUDA tensors; there is no CPU path")
        now = self._tensor_amax(x)
        if self.amax_history.numel() == 0 or self.amax_history.dtype != x.dtype:
            self._allocate(now.shape, x.dtype, x.device)
        channels = self.scale.numel()
        N.check(N.lib().vq_amax_history_update(self.amax_history.data_ptr(), _dtype_id(x.dtype), self.amax_history_len,
                                               channels, self.ring_position.data_ptr(), now.data_ptr(),
                                               _dtype_id(now.dtype), now.numel(), float(self.quant_max),
                                               int(self.power_2_scale), self.scale.data_ptr(), _stream()),
                "vq_amax_history_update")

    # the reference's name for the same step
    _update_amax_scale = observe

    def calculate_qparams(self):
        return self.scale

    @N.device_guarded
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._observe:
            self.observe(x)
        if not self._quantize:
            return x
        return torch.ops.quantization.fake_quant(x, self.qmap, self.scale)

    def extra_repr(self):
        return (f"dtype={self.dtype}, qscheme={self.qscheme}, quant_max={self.quant_max}, ch_axis={self.ch_axis}, "
                f"amax_history_len={self.amax_history_len}, power_2_scale={self.power_2_scale}")
