"""B200-native inference runtime with the capability set of CoffeeVampir3/Mojo-Linuxperiments.

Layers (bottom up):
  hostrt   C++ host runtime: raw syscalls, NUMA topology, CPU masks, NUMA arena, clone3/futex worker pool
  devrt    GPU/NVLink topology, device masks, HBM arenas, symmetric (peer-mapped) memory
  ops      hand-written sm_100a kernels (tcgen05 + TMEM + TMA) behind thin Python wrappers
  parallel tensor/expert-parallel layers whose collectives run inside the compute kernels
  models   Llama-shaped dense and Qwen3-shaped MoE decoders, int8 weight + scale checkpoints
  engine   paged KV cache, CUDA-graph decode loop, greedy sampling
"""
__version__ = "0.1.0"
