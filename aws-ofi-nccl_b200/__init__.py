"""B200-native NCCL transport framework: net/tuner/GIN plugin + fused sm_100a kernels.

Sub-packages
  ops       ctypes bindings of the hand-written CUDA kernels (libb200ops.so)
  parallel  symmetric memory, device collectives, DP / TP / EP building blocks
  models    Llama-3 training model, tensor-parallel MLP, MoE layer
  utils     timing, clock sampling, checkpointing, tuner inspection CLI
The C++ plugin that NCCL loads lives in ``csrc/`` and is built by ``build.py``.
"""
__version__ = "0.1.0"
