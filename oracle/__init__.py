"""CPU oracle of the column-reduction operator.

TEST INFRASTRUCTURE ONLY.  Nothing under ``oracle/`` is part of the product:
only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference
legs of ``bench.py`` may import or execute it, and only as the checker or the
timed CPU baseline -- never on the path a user of the library runs.
"""
from .colreduce_oracle import oracle_colreduce, oracle_valid_scores  # noqa: F401
