"""CPU oracle for the embedding-extraction path: TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may
import this package; the shipped library never does.
"""
