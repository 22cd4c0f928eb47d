"""kb_nano_b200 -- B200 (sm_100a) implementation of kb-nano's FP8 W8A8 hot path.

  ops        tensor-level calls into the C-ABI CUDA library (libkbn_fp8.so)
  torch_ops  the same calls registered as opaque torch.library ops (for torch.compile)
  candidate  drop-in modules for kb-nano's tasks/candidate + infra/kernel_swapper interface
  inputs     seeded synthetic inputs of the benchmark configurations
  build      in-tree nvcc build of the library
"""
from . import _lib, ops  # noqa: F401

__all__ = ["ops", "candidate_dir", "install_candidates"]


def candidate_dir() -> str:
    """Directory to point $KB_NANO_CANDIDATE_DIR at."""
    import os
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "candidate")
