"""B200-native path of MiniWorld's Pairformer triangle multiplicative update (forward; backward of the unidirectional
module in :mod:`miniworld_b200.training`).

Public surface: the module classes (drop-in for ``miniworld_engine.modules.TriangleMultiplication`` as
MiniWorld's blocks use it), the functional entry points over the C ABI, and the row-sharded /
batch-parallel multi-GPU wrappers.
"""

from .modules import (  # noqa: F401
    BidirectionalTriangleMultiplication,
    Transition,
    TriangleMultiplication,
    TriangleMultiplicationIncoming,
    TriangleMultiplicationOutgoing,
    from_openfold_state_dict,
    to_openfold_state_dict,
)

__all__ = [
    "TriangleMultiplication",
    "BidirectionalTriangleMultiplication",
    "Transition",
    "TriangleMultiplicationOutgoing",
    "TriangleMultiplicationIncoming",
    "to_openfold_state_dict",
    "from_openfold_state_dict",
]
