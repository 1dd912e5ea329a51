"""CPU oracle for the decode hot path: TEST INFRASTRUCTURE ONLY.

Imported by tests/, by the smoke check and by the benchmark's CPU-baseline leg;
never by the product package.
"""
