"""Import path of the 8-bit quantisation hooks (ddp_comm_hooks/quantization_hooks.py in the reference)."""
from ... import algorithms as _a

quantization_pertensor_hook, quantization_perchannel_hook = _a.quantization_pertensor_hook, _a.quantization_perchannel_hook
