"""CPU oracle of the reference's operator math.  TEST INFRASTRUCTURE ONLY.

Nothing under ``heron_b200/`` imports this package; the test-suite, the smoke check and the
benchmark's cpu-baseline / reference legs are its only callers.
"""
