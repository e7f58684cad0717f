"""B200-native TriangleMultiplication block (hand-written sm_100a kernels behind a C ABI).

Public surface:

* ``TriangleMultiplicationB200`` — ``nn.Module`` with the reference module's interface;
* ``triangle_multiplicative_update_b200`` — the reference's functional signature;
* ``BidirectionalTriangleMultiplicationB200`` / ``bidir_trimul_forward`` /
  ``bidirectional_triangle_multiplicative_update_b200`` — the reference's bidirectional block
  (outgoing and incoming contraction on the two halves of a doubled hidden width), as module, with
  this package's argument names and with those of the reference's functional op;
* ``install`` / ``from_reference`` — replace the reference's triangle-multiplication modules of an
  already-built model by their B200 twins (same parameters and ``state_dict`` keys).

The compiled library ``libtrimul_b200.so`` is the only compute path; importing this
package does not load it, the first call does, and a missing library raises.
"""

from .functional import read_status, triangle_multiplicative_update_b200, trimul_forward, workspace_bytes
from .convert import from_reference, install
from .bidirectional import (BidirectionalTriangleMultiplicationB200, bidir_trimul_forward,
                            bidirectional_triangle_multiplicative_update_b200)
from .module import TriangleMultiplicationB200

__all__ = [
    "TriangleMultiplicationB200",
    "BidirectionalTriangleMultiplicationB200",
    "bidir_trimul_forward",
    "bidirectional_triangle_multiplicative_update_b200",
    "install",
    "from_reference",
    "triangle_multiplicative_update_b200",
    "trimul_forward",
    "read_status",
    "workspace_bytes",
]
