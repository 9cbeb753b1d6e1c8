"""eps_b200: the FP8 MoE expert-layer path of meituan-longcat/eps for B200 (sm_100a).

Importing the package does not load the CUDA library; the first operator call does, and raises if
`libeps_b200.so` has not been built (`python -m eps_b200.build`).  There is no CPU fallback.
"""
__all__ = ["ops", "scheduler", "executor", "fast_ep", "communication", "layer", "workloads"]
