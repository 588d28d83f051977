"""B200 (sm_100a) implementation of the chunked XMC classifier layer of xmc-aalto/elmo.

``elmo_b200.xmc_classifiers`` mirrors the reference's ``src/xmc_classifiers`` package (same class
names, constructor and methods); the arithmetic runs in the CUDA library behind
``include/elmo_xmc.h``.
"""
__all__ = ["xmc_classifiers", "handle", "synth"]
