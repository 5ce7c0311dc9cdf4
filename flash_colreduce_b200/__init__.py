"""flash_colreduce for NVIDIA B200 (sm_100a).

Drop-in for the Python API of z-lab/flash-colreduce
(flash_colreduce/__init__.py:1-4): ``flash_colreduce``, ``naive_colreduce``
and ``__version__``.
"""
from .dense import naive_colreduce
from .host import flash_colreduce_host
from .op import colreduce_partial, finalize_scores, flash_colreduce, flash_colreduce_topk, select_columns, topk_columns, valid_scores

__version__ = "0.1.0"
__all__ = ["flash_colreduce", "naive_colreduce", "colreduce_partial", "finalize_scores", "valid_scores",
           "flash_colreduce_host", "topk_columns", "flash_colreduce_topk", "select_columns",
           "__version__"]
