"""B200 (sm_100a) implementation of the 4-bit MoE hot path of fbundle/moe_infer.

``moe_infer_b200.native``  object wrapper over the C ABI (include/moe_b200.h)
``moe_infer_b200._moe_infer_rs``  mirror of the reference's PyO3 module surface
``moe_infer_b200.build``   in-tree nvcc build of libmoe_b200.so

The compute path is the CUDA library only; there is no CPU fallback.
"""
__all__ = ["native", "build"]
