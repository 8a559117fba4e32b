"""rl_engine: a Blackwell-native (sm_100a) operator library for RL post-training.

Public surface mirrors the RL-Kernel project layout (``rl_engine.kernels.registry``,
``rl_engine.kernels.sampling``, ``rl_engine.executors`` ...), while every GPU hot path is a
hand-written sm_100a kernel living in the in-tree extension ``rl_engine._C``.
"""

__version__ = "0.1.0"
