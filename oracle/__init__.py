"""TEST INFRASTRUCTURE ONLY: CPU restatement of the reference's chunked XMC classifier step.

Imported by tests/, by the smoke check and by the CPU-baseline legs of bench.py -- never by the
product package.
"""
