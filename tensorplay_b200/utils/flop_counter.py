"""``utils.flop_counter``: PyTorch's ``FlopCounterMode`` extended to the native kernels.

PyTorch's counter is a dispatch mode: it sees ATen operators. The GEMMs, attention and grouped GEMMs of this
package are launched through a C ABI from autograd functions and never reach the dispatcher, so the stock
counter reports a model built from them as (almost) free. The op wrappers therefore report each launch's
floating-point work to ``_native.add_flops``; the mode here registers itself as a sink while it is active and
books that work under the module that is running, next to the ATen operators it counts itself
(tensorplay/utils/flop_counter.py: ``FlopCounterMode``; the formulas are those of its registry: 2 M N K for a
product, four products of B H Tq Tk D for attention forward with a causal square counted half, ten backward).
"""
from torch.utils.flop_counter import *  # noqa: F401,F403
from torch.utils.flop_counter import FlopCounterMode as _TorchFlopCounterMode

from .. import _native


class FlopCounterMode(_TorchFlopCounterMode):
    def __enter__(self):
        out = super().__enter__()
        _native.flop_sinks.append(self._native_flops)
        return out

    def __exit__(self, *args):
        try:
            _native.flop_sinks.remove(self._native_flops)
        except ValueError:
            pass
        return super().__exit__(*args)

    def _native_flops(self, name: str, flops: int) -> None:
        for parent in set(self.mod_tracker.parents):
            self.flop_counts[parent][name] += flops
