"""Literal inputs held by the reference's own smoke harnesses (inputs only: the reference
commits no expected outputs; its harnesses print results or recompute them with PyTorch)."""
import numpy as np

# examples/torch/layernorm/cuda/layernorm.cu:24-26 — fp32 [2, 10]
LAYERNORM_2x10 = np.array(
    [0.8823, 0.9150, 0.3829, 0.9593, 0.3904, 0.6009, 0.2566, 0.7936, 0.9408, 0.1332,
     0.9346, 0.5936, 0.8694, 0.5677, 0.7411, 0.4294, 0.8854, 0.5739, 0.2666, 0.6274],
    dtype=np.float32).reshape(2, 10)

# examples/torch/elementwise/add.cu:21-26 — fp32 [3, 3, 3] + [3, 1, 3]
ADD_A_3x3x3 = np.array(
    [0.8823, 0.9150, 0.3829, 0.9593, 0.3904, 0.6009, 0.2566, 0.7936, 0.9408,
     0.1332, 0.9346, 0.5936, 0.8694, 0.5677, 0.7411, 0.4294, 0.8854, 0.5739,
     0.2666, 0.6274, 0.2696, 0.4414, 0.2969, 0.8317, 0.1053, 0.2695, 0.3588],
    dtype=np.float32).reshape(3, 3, 3)
ADD_B_3x1x3 = np.array([0.1994, 0.5472, 0.0062, 0.9516, 0.0753, 0.8860, 0.5832, 0.3376, 0.809],
                       dtype=np.float32).reshape(3, 1, 3)

# examples/torch/bert_attention/cuSeqLen.cu:26-33 — valid lengths, repeated for bs 16, seq 64
CU_SEQLEN_VALID_LENGTHS = [64, 12, 31, 32, 33, 34, 35, 36]
