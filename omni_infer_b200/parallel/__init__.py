"""Process groups, NCCL/gloo communicators, the NVLink symmetric heap and the fused
compute+collective kernels' host side."""
from .parallel_state import (GroupCoordinator, ParallelState, destroy_distributed, get_parallel_state,  # noqa: F401
                             init_distributed)
