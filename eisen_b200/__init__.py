"""eisen_b200: B200-native (sm_100a) training-step hot path behind the Eisen Graph API.

The package is a thin host-side mirror over libeisen_b200.so (CUDA kernels + C ABI).  Importing
it does not need a GPU; any compute call does, and fails loudly without one.
"""
from ._lib import EisenError, call, check, declarations, lib  # noqa: F401

F32 = 0
BF16 = 1
