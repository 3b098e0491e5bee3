"""CUDA sources of the kernels (sm_100a) and the script that builds them into one library."""
from .build import library_path, build

__all__ = ["library_path", "build"]
