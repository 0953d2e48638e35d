"""CPU oracle (test infrastructure, not product code).

Only the test-suite, the smoke check and the CPU leg of the benchmark may
import from here.  See ``sdpa_oracle.py``.
"""
