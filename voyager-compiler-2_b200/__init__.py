"""B200-native (sm_100a) kernels behind voyager_compiler's ``quantized_ops`` operators.

Importing the package registers the ``quantized_ops`` torch library with CUDA
kernels (see ``ops``).  The directory name is not a Python identifier; import
it through the ``voyager_b200`` module at the repository root.
"""

from . import _native, formats, rounding  # noqa: F401
from . import ops  # noqa: F401  (registers torch.ops.quantized_ops.*)
from . import fp8  # noqa: F401
from . import workloads  # noqa: F401
from . import gptq  # noqa: F401
from . import parallel  # noqa: F401
from . import nvfp4  # noqa: F401
from . import fake_quant  # noqa: F401  (registers torch.ops.quantization.*)
from . import kivi  # noqa: F401
from . import packed  # noqa: F401
from . import training  # noqa: F401  (registers torch.ops.voyager_gpu.rmsnorm_backward)
from . import observers  # noqa: F401
from . import outliers  # noqa: F401  (adds the outlier operators to torch.ops.quantized_ops)
from ._native import build  # noqa: F401
from .formats import (  # noqa: F401
    QScheme,
    entry_levels,
    float_format,
    get_quantization_map,
    int_range,
    parse_codebook_dtype,
    parse_spec_fields,
    posit_format,
    qmap_levels,
)
from .ops import calculate_global_scale, tensor_amax  # noqa: F401
