"""B200-native GRPO loss boundary: Python binding of ``libgrpo_b200.so``.

The product is the shared library (hand-written sm_100a CUDA kernels behind a C ABI, declared in
``include/grpo_b200.h``, plus C++ wrappers with the reference's ``namespace grpo`` signatures).
This package binds the C ABI with ``ctypes`` so that tests and benchmarks can drive it:

* :mod:`.api` -- the reference-facing calls under the reference's own names
  (``grpo_loss_cuda``, ``grpo_logits_cuda``, ``grpo_logits_cuda_device_inplace``,
  ``benchmark_grpo_loss_cuda``, ``benchmark_grpo_logits_cuda``; reference
  include/grpo/grpo_loss_cuda.cuh:26-102) taking numpy arrays where the reference takes
  ``std::vector``;
* :mod:`.device` -- the device layer on ``torch`` CUDA tensors (memory and streams only; no
  torch op is on the compute path);
* :mod:`.sharded` -- token-sharded execution over ``torch.distributed``;
* :mod:`.workloads` -- seeded synthetic inputs of the benchmark configurations.

There is no CPU or eager fallback: importing works anywhere (so the library's symbols can be
inspected), but every compute call needs the CUDA library and a device and fails loudly otherwise.
"""
from ._lib import LIB_PATH, build, lib, last_error  # noqa: F401
from .api import (  # noqa: F401
    AdvantageMode,
    CudaLogitsKernel,
    CudaLogitsTiming,
    CudaLossKernel,
    CudaTiming,
    LogitsLossResult,
    LossConfig,
    LossResult,
    LossStats,
    ReductionMode,
    benchmark_grpo_logits_cuda,
    benchmark_grpo_loss_cuda,
    grpo_logits_cuda,
    grpo_logits_cuda_device_inplace,
    grpo_loss_cuda,
)

__all__ = [
    "AdvantageMode", "CudaLogitsKernel", "CudaLogitsTiming", "CudaLossKernel", "CudaTiming",
    "LogitsLossResult", "LossConfig", "LossResult", "LossStats", "ReductionMode",
    "benchmark_grpo_logits_cuda", "benchmark_grpo_loss_cuda", "grpo_logits_cuda",
    "grpo_logits_cuda_device_inplace", "grpo_loss_cuda", "build", "lib", "last_error", "LIB_PATH",
]
