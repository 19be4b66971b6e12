"""Q38 sparse-MoE pretraining framework for NVIDIA B200 (sm_100a).

Sub-packages and modules
  models/    module tree + PyTorch specification of every op (also the HF remote-code file)
  ops/       Python bindings and autograd wrappers of the hand-written CUDA kernels (csrc/)
  optim/     Muon + AdamW hybrid optimizer, fused update kernels
  parallel/  peer-memory gradient engine, owner-computes optimizer sharding, expert parallelism
  utils/     timing, NVTX, clocks sampling, synthetic streams, checkpoint helpers
  presets, flops, data, sampling   configuration, accounting and data plumbing
  train, evaluate                   entry points: python -m q38.train / q38.evaluate / q38.flops / q38.data
"""
__version__ = "0.1.0"
