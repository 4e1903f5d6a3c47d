"""Delayed-scaling fake-quantizer for the per-tensor and per-channel schemes on the CUDA kernels.

Mirror of the reference's ``FusedAmaxObsFakeQuantize``
(``src/voyager_compiler/quantization/fake_quantize.py:330-447``): same constructor
arguments, buffers (``qmap``, ``scale``, ``amax_history``) and methods.  The module keeps
the absolute maxima of the last ``amax_history_len`` inputs, one per tensor or one per
channel along ``ch_axis``, and scales by the largest; an input is quantized before its own
amax joins the history, so the first call uses scale 1.  History and scale take the dtype of
the tensor quantized.  The amax of a whole tensor is one pass of ``vq_amax``; the
fake-quantize is ``torch.ops.quantization.fake_quant``.
"""

from typing import Optional, Tuple

import torch

from .formats import QScheme, get_quantization_map
from .ops import tensor_amax


class FusedAmaxObsFakeQuantize(torch.nn.Module):
    def __init__(self, dtype: str, qscheme: QScheme, quant_max: float, amax_history_len: int,
                 ch_axis: Optional[int] = None, power_2_scale: bool = False, device=None, **unused) -> None:
        if qscheme not in (QScheme.PER_TENSOR_SYMMETRIC, QScheme.PER_CHANNEL_SYMMETRIC):
            raise ValueError(f"{qscheme} is not a per-tensor or per-channel scheme")
        super().__init__()
        self.dtype = dtype
        self.qscheme, self.quant_max = qscheme, quant_max
        self.amax_history_len, self.ch_axis, self.power_2_scale = amax_history_len, ch_axis, power_2_scale
        self.is_per_channel = qscheme == QScheme.PER_CHANNEL_SYMMETRIC
        self.register_buffer("qmap", get_quantization_map(dtype, device), persistent=False)
        self.register_buffer("scale", torch.tensor([1.0], dtype=torch.float, device=device))
        self.register_buffer("amax_history", torch.tensor([], dtype=torch.float, device=device))
        self.register_buffer("fake_quant_enabled", torch.tensor([1], dtype=torch.uint8))
        self.register_buffer("observer_enabled", torch.tensor([1], dtype=torch.uint8))
        self._observe, self._quantize = True, True

    # the enable switches are host flags as well, so that forward never reads a device value
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

    def start_history(self, shape: Tuple[int, ...], dtype) -> None:
        """Size the history and the scale as before any input (``fake_quantize.py:389-403``)."""
        device = self.scale.device
        self.amax_history = torch.zeros((self.amax_history_len, *shape), dtype=dtype, device=device)
        self.scale = torch.ones(shape, dtype=dtype, device=device)

    @torch.no_grad()
    def _update_amax_scale(self, x: torch.Tensor) -> None:
        """Recompute ``scale`` from the history, then fold ``x``'s amax into the history
        (``fake_quantize.py:406-437``)."""
        if self.is_per_channel:
            ch_axis = self.ch_axis % x.ndim
            dim = tuple(i for i in range(x.ndim) if i != ch_axis)
            amax_cur = torch.amax(torch.abs(x), dim=dim, keepdim=True)
        elif x.is_cuda:
            amax_cur = tensor_amax(x).to(x.dtype)        # one pass, no |x| temporary
        else:
            amax_cur = torch.amax(torch.abs(x))
        if self.amax_history.numel() == 0:
            self.start_history(amax_cur.shape, x.dtype)
        amax = torch.amax(self.amax_history, dim=0)
        self.amax_history.copy_(torch.roll(self.amax_history, -1, 0))
        self.amax_history[0] = amax_cur
        sf = amax / self.quant_max
        sf = torch.where(amax > 0.0, sf, self.scale)
        sf = torch.where(torch.isfinite(amax), sf, self.scale)
        if self.power_2_scale:
            sf = torch.pow(2, torch.ceil(torch.log2(sf)))
        self.scale.copy_(sf)

    def calculate_qparams(self):
        return self.scale

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._observe:
            self._update_amax_scale(x)
        if not self._quantize:
            return x
        return torch.ops.quantization.fake_quant(x, self.qmap, self.scale)

    def extra_repr(self):
        return (f"dtype={self.dtype}, qscheme={self.qscheme}, quant_max={self.quant_max}, ch_axis={self.ch_axis}, "
                f"amax_history_len={self.amax_history_len}, power_2_scale={self.power_2_scale}")
