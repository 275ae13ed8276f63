"""B200 (sm_100a) sigmoid attention: a drop-in for the Python API of triton-sigmoid.

    from triton_sigmoid_b200 import sigmoid_attention, sigmoid_attention_padded

Both functions run hand-written CUDA kernels through a C-ABI shared library
(``include/sigattn_b200.h``); there is no Triton, no backend dispatch and no CPU path.
``sigmoid_attention_varlen`` is the same computation on packed variable-length sequences (not in
the reference).  ``sigmoid_attention_ref`` is the plain PyTorch formula, exported because the reference
package exports one too; it is not used by the two functions above.

Run-time switches: ``TRITON_SIGMOID_ACCURATE=1`` (the reference's variable, read at every call) or the
``accurate_sigmoid()`` context manager select the accurate sigmoid; ``SIGATTN_B200_DEBUG=1`` makes every
call synchronise and raise if a kernel gave up on one of its bounded waits; ``device_status()`` reads
and clears that health word on demand.
"""

__version__ = "0.1.0"

from .ops import (accurate_sigmoid, device_status, sigmoid_attention, sigmoid_attention_padded,
                  sigmoid_attention_varlen)
from .reference_math import sigmoid_attention_ref

__all__ = [
    "sigmoid_attention",
    "sigmoid_attention_padded",
    "sigmoid_attention_varlen",
    "sigmoid_attention_ref",
    "accurate_sigmoid",
    "device_status",
]
