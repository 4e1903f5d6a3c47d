"""Import the reference's CPU ops from a read-only checkout, without editing it.

Used only by ``make_golden.py`` (fixture generation) and by the optional
"live reference" parity tests; nothing on the product path imports this.

The reference package cannot be imported whole in an environment that has
torch 2.11 and no torchao, so three harness-side shims are installed first:

1. ``torch.compile`` is wrapped so that unknown keyword arguments
   (``recompile_limit``) are dropped and the function is returned unchanged:
   on CPU the reference runs its ops as written, which is the behaviour the
   fixtures pin (``src/voyager_compiler/ops/quantized.py:41-60``).
2. Stub parent packages ``voyager_compiler`` and
   ``voyager_compiler.quantization`` (with ``__path__`` pointing into the
   checkout) are pre-registered so their ``__init__`` modules, which import
   torchao transitively, never run.
3. A stub ``torchao.quantization.pt2e`` exposing ``FakeQuantizeBase`` and
   ``ObserverOrFakeQuantize`` lets ``quantization/fake_quantize.py`` import
   (its lookup tables are what we need), and a stub
   ``voyager_compiler.quantization.codebook_optimizer`` exposing ``EPS`` lets
   ``quantization/gptq.py`` import.

The reference registers ``Library("quantized_ops", "DEF")``; a process that
has loaded the reference therefore must not also load this repository's op
boundary.  The golden generator runs in its own process for that reason.
"""

import importlib
import os
import sys
import types

import torch

# The checkout is named by the environment alone; without the variable the reference is "not available".
REFERENCE_ROOT = os.environ.get("VOYAGER_REFERENCE_ROOT", "")
_SRC = os.path.join(REFERENCE_ROOT, "src")


def available() -> bool:
    return bool(REFERENCE_ROOT) and os.path.isdir(os.path.join(_SRC, "voyager_compiler", "ops"))


def _install_shims():
    if getattr(torch.compile, "_vq_shimmed", False):
        return

    def tolerant_compile(fn=None, **kwargs):
        if fn is None:
            return lambda f: f
        return fn

    tolerant_compile._vq_shimmed = True
    torch.compile = tolerant_compile

    pkg_root = os.path.join(_SRC, "voyager_compiler")
    for name, path in (
        ("voyager_compiler", pkg_root),
        ("voyager_compiler.quantization", os.path.join(pkg_root, "quantization")),
    ):
        module = types.ModuleType(name)
        module.__path__ = [path]
        sys.modules[name] = module

    torchao = types.ModuleType("torchao")
    torchao.__path__ = []
    tq = types.ModuleType("torchao.quantization")
    tq.__path__ = []
    pt2e = types.ModuleType("torchao.quantization.pt2e")

    class FakeQuantizeBase(torch.nn.Module):
        def __init__(self, *args, **kwargs):
            super().__init__()
            self.register_buffer("fake_quant_enabled", torch.tensor([1], dtype=torch.uint8))
            self.register_buffer("observer_enabled", torch.tensor([1], dtype=torch.uint8))

    pt2e.FakeQuantizeBase = FakeQuantizeBase
    pt2e.ObserverOrFakeQuantize = object
    sys.modules.setdefault("torchao", torchao)
    sys.modules.setdefault("torchao.quantization", tq)
    sys.modules.setdefault("torchao.quantization.pt2e", pt2e)

    cb = types.ModuleType("voyager_compiler.quantization.codebook_optimizer")
    cb.EPS = 1e-12  # src/voyager_compiler/quantization/codebook_optimizer.py:51
    sys.modules["voyager_compiler.quantization.codebook_optimizer"] = cb


class Reference:
    """Handles to the reference modules that define the hot path."""

    def __init__(self):
        if not available():
            raise RuntimeError("set VOYAGER_REFERENCE_ROOT to a checkout of the reference (found none at "
                               f"{REFERENCE_ROOT!r})")
        _install_shims()
        self.ops = importlib.import_module("voyager_compiler.ops")
        self.quantized = importlib.import_module("voyager_compiler.ops.quantized")
        self.layout = importlib.import_module("voyager_compiler.ops.layout")
        self.qspec = importlib.import_module("voyager_compiler.quantization.qspec")
        self.mx_utils = importlib.import_module("voyager_compiler.quantization.mx_utils")
        self.dtypes = importlib.import_module("voyager_compiler.quantization.dtypes")
        self._fake_quantize = None
        self._gptq = None

    @property
    def fake_quantize(self):
        if self._fake_quantize is None:
            self._fake_quantize = importlib.import_module(
                "voyager_compiler.quantization.fake_quantize"
            )
        return self._fake_quantize

    @property
    def gptq(self):
        if self._gptq is None:
            self._gptq = importlib.import_module("voyager_compiler.quantization.gptq")
        return self._gptq


_REFERENCE = None


def load() -> Reference:
    global _REFERENCE
    if _REFERENCE is None:
        _REFERENCE = Reference()
    return _REFERENCE
