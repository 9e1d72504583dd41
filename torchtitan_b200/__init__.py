"""torchtitan_b200: a Blackwell-native LLM pre-training framework.

PyTorch is the tensor/autograd layer; the hot operators are hand-written
sm_100a CUDA kernels (``torchtitan_b200.ops``) and the sharded-data-parallel
engine, tensor/context/expert/pipeline parallelism live in
``torchtitan_b200.parallel``.
"""

__version__ = "0.1.0"
