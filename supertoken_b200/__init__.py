"""B200-native BPE merge-loop engine behind the reference's ``GPUBPETrainer`` API.

The CUDA library (``libstbpe.so``, sm_100a) is required; nothing here falls back to a CPU
implementation."""
from .bpe_trainer import GPUBPETrainer  # noqa: F401

__all__ = ["GPUBPETrainer"]
