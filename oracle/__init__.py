"""CPU oracle for the JGPT KV-cache decode path: test infrastructure only.

Nothing in ``jgpt_b200`` imports this package.  It is used by ``tests/``, by the smoke
check and by the CPU-baseline leg of ``bench.py`` as the checker the CUDA path is compared with.
"""
from .oracle import *  # noqa: F401,F403
