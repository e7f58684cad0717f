"""B200-native TriangleMultiplication block (hand-written sm_100a kernels behind a C ABI).

Public surface:

* ``TriangleMultiplicationB200`` — ``nn.Module`` with the reference module's interface;
* ``triangle_multiplicative_update_b200`` — the reference's functional signature;
* ``BidirectionalTriangleMultiplicationB200`` / ``bidir_trimul_forward`` — the reference's
  bidirectional block (outgoing and incoming contraction on the two halves of a doubled hidden width);
* ``install`` — registers the backend on an imported reference package.

The compiled library ``libtrimul_b200.so`` is the only compute path; importing this
package does not load it, the first call does, and a missing library raises.
"""

from .functional import read_status, triangle_multiplicative_update_b200, trimul_forward, workspace_bytes
from .bidirectional import BidirectionalTriangleMultiplicationB200, bidir_trimul_forward
from .module import TriangleMultiplicationB200

__all__ = [
    "TriangleMultiplicationB200",
    "BidirectionalTriangleMultiplicationB200",
    "bidir_trimul_forward",
    "triangle_multiplicative_update_b200",
    "trimul_forward",
    "read_status",
    "workspace_bytes",
]
