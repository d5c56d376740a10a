"""CPU oracle for the brute.bit1 hot path -- TEST INFRASTRUCTURE ONLY.

``oracle.c_oracle`` wraps the C restatement (``brute_oracle.c``) through ctypes
on numpy arrays; ``oracle.np_oracle`` restates the same functions a second time
in plain numpy for cross-checking at small sizes. Nothing in the ``brute_b200``
package imports this module: only tests, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` do, and only as the
checker or the timed CPU baseline.
"""
