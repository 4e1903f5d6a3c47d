"""CPU restatement of the reference's delayed-scaling observer (test infrastructure only).

``FusedAmaxObsFakeQuantize`` (reference ``src/voyager_compiler/quantization/fake_quantize.py:330-447``)
keeps the absolute maxima of the last ``amax_history_len`` inputs and scales by the largest;
an input is quantized before its own amax joins the history, so the first call uses scale 1.
Pinned by the golden cases ``observer_*``, produced by feeding sequences through the reference
module itself.
"""

import torch

from . import fake_quant as FQ
from . import tables as T


class AmaxObserver:
    def __init__(self, dtype, quant_max, history_len, ch_axis=None, power_2_scale=False):
        self.qmap = T.quantization_map(dtype)
        self.quant_max, self.history_len = quant_max, history_len
        self.ch_axis, self.power_2_scale = ch_axis, power_2_scale
        self.history = None
        self.scale = torch.tensor([1.0])

    def update(self, x):
        """``_update_amax_scale`` (reference ``fake_quantize.py:406-437``)."""
        if self.ch_axis is not None:
            ch = self.ch_axis % x.ndim
            amax_cur = torch.amax(torch.abs(x), dim=tuple(i for i in range(x.ndim) if i != ch), keepdim=True)
        else:
            amax_cur = torch.amax(torch.abs(x))
        if self.history is None:
            self.history = torch.zeros((self.history_len, *amax_cur.shape), dtype=x.dtype)
            self.scale = torch.ones(amax_cur.shape, dtype=x.dtype)
        amax = torch.amax(self.history, dim=0)
        self.history = torch.roll(self.history, -1, 0)
        self.history[0] = amax_cur
        sf = amax / self.quant_max
        sf = torch.where(amax > 0.0, sf, self.scale)
        sf = torch.where(torch.isfinite(amax), sf, self.scale)
        if self.power_2_scale:
            sf = torch.pow(2, torch.ceil(torch.log2(sf)))
        self.scale = sf.to(self.scale.dtype)

    def __call__(self, x):
        self.update(x)
        return FQ.fake_quant(x, self.qmap, self.scale)


def amax_observer(sequence, dtype, quant_max, history_len, ch_axis, power_2_scale):
    """Outputs and scales after each element of ``sequence`` went through one observer."""
    obs = AmaxObserver(dtype, quant_max, history_len, ch_axis, power_2_scale)
    outs, scales = [], []
    for x in sequence:
        outs.append(obs(x))
        scales.append(obs.scale.clone())
    return torch.stack(outs), torch.stack(scales)
