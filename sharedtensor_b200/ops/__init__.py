from .table import SharedTable, TableLayout, createOrFetchTable

__all__ = ["SharedTable", "TableLayout", "createOrFetchTable"]
