"""CPU restatement of the reference SQAttn arithmetic.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; it is used by the test-suite, by the smoke check and by the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark as the checker
and as the timed CPU baseline.
"""
