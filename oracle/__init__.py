"""TEST INFRASTRUCTURE ONLY: CPU restatement of the reference's host MoE path.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this package; the product library never does.
"""
