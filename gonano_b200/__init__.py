"""gonano_b200: a B200-native CUDA backend for gonano's RL step.

The product is the C-ABI shared library built from ``gonano_b200/csrc``
(``include/gonano_cuda.h``); this package is its Python host-side mirror of the
reference interface (``kernels.Backend``, ``inference.Engine``, ``trainer.RLStep``).
"""
