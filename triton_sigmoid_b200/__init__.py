"""B200 (sm_100a) sigmoid attention: a drop-in for the Python API of triton-sigmoid.

    from triton_sigmoid_b200 import sigmoid_attention, sigmoid_attention_padded

Both functions run hand-written CUDA kernels through a C-ABI shared library
(``include/sigattn_b200.h``); there is no Triton, no backend dispatch and no CPU path.
``sigmoid_attention_varlen`` is the same computation on packed variable-length sequences (not in
the reference).  ``sigmoid_attention_ref`` is the plain PyTorch formula, exported because the reference
package exports one too; it is not used by the two functions above.
"""

__version__ = "0.1.0"

from .ops import sigmoid_attention, sigmoid_attention_padded, sigmoid_attention_varlen
from .reference_math import sigmoid_attention_ref

__all__ = [
    "sigmoid_attention",
    "sigmoid_attention_padded",
    "sigmoid_attention_varlen",
    "sigmoid_attention_ref",
]
