"""FlexTree for B200: tree all-reduce over NVLink peer memory, n-way reduction kernels,
tree-width cost model and an MPI_Allreduce-style entry point.

Sub-packages
    ops       n-way reduce kernels (single GPU) and their CPU oracle
    parallel  planner / cost model bindings, the multi-GPU communicator, the CPU worlds (ranks as threads or as
              processes of one host), DDP integration, calibration, a one-host launcher
    models    GPT-2 used by the data-parallel benchmark
    utils     logging, timing, clock sampling
"""
from ._lib import FlexTreeError, lib  # noqa: F401

__version__ = "0.1"
