"""hiptensor_b200: host-side mirror of the hipTensor interface for the contraction,
permutation and reduction paths, over hand-written sm_100a CUDA kernels.

The compute path is libhiptensor_b200.so (C++/CUDA, built in-tree by
`python -m hiptensor_b200.build`); this package only marshals arguments through the flat C
ABI declared in include/hiptensor_b200.h. Names and argument meaning follow
ROCm/hipTensor's library/include/hiptensor/hiptensor.hpp.
"""
from .api import *  # noqa: F401,F403
from .api import __all__  # noqa: F401
