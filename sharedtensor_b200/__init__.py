"""sharedtensor_b200 — an asynchronous, eventually consistent, replicated fp32 tensor for B200 boxes.

Same API and tree-join protocol as Hello1024/shared-tensor (``createOrFetch``, ``copyToTensor``,
``addFromTensor``), re-designed around GPU-resident replicas that exchange 1-bit, block-scaled,
error-feedback deltas through peer memory over NVLink.
"""
from .api import SharedTensor, createOrFetch
from .ops.table import SharedTable, createOrFetchTable
from .utils.config import Config

__all__ = ["SharedTensor", "createOrFetch", "SharedTable", "createOrFetchTable", "Config"]
__version__ = "0.1.0"
