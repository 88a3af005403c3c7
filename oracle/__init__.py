"""CPU oracle for the training hot path (test infrastructure only).

Nothing in the product package imports this module. It is used by ``tests/``, by
``__graft_entry__.smoke()`` and by ``bench.py``'s CPU-baseline leg as the checker.
"""
from .binding import (  # noqa: F401
    STATE_STORAGE_LEN,
    MlpShape,
    Oracle,
    Reference,
    build_oracle,
    load_oracle,
    load_reference,
)
