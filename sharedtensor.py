"""``import sharedtensor`` — the module name the reference is loaded under (``require 'sharedtensor'``,
example.lua:2).  Everything lives in :mod:`sharedtensor_b200`."""
from sharedtensor_b200 import Config, SharedTable, SharedTensor, createOrFetch, createOrFetchTable  # noqa: F401

__all__ = ["createOrFetch", "createOrFetchTable", "SharedTensor", "SharedTable", "Config"]
