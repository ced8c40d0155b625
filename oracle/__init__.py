"""CPU restatement of the reference's FP8 preparation and ExpCast attention.

TEST INFRASTRUCTURE ONLY. Nothing in the shipped package imports this module;
only the tests, the smoke check and the benchmark's CPU-baseline leg call it,
and only as the checker.
"""
