"""forja_b200: B200-native (sm_100a) backend for forja's continuous-batching forward step.

The product is the C-ABI shared library ``libforja_cuda.so`` (sources in ``csrc/``, interface in
``include/forja_cuda.h``). This package holds the build recipe and a thin ctypes mirror of the
reference's backend interface used by tests and benchmarks. Importing it never touches a CPU
fallback: every compute entry point needs the compiled library and a CUDA device.
"""
from .backend import (BF16, F16, F32, I32, U32, BackendError, CommandList, CudaBackend, DenseModel, ExpertParallel, KvPool, Layout,
                      MoeModel, Op, Submission, Tensor)
from .scheduler import SchedulerPolicy, chunk_merged_work, chunk_work, prefill_plan, reservations_fit

__all__ = ["BF16", "F16", "F32", "I32", "U32", "BackendError", "CommandList", "CudaBackend", "DenseModel", "KvPool", "Layout",
           "Op", "Submission", "Tensor", "ExpertParallel", "MoeModel", "SchedulerPolicy", "chunk_work", "chunk_merged_work", "prefill_plan", "reservations_fit"]
