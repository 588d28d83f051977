"""TEST INFRASTRUCTURE ONLY -- CPU restatement of the Philox4x32 counter-based RNG.

The algorithm is the published one (Salmon et al., "Parallel random numbers: as easy as
1, 2, 3", SC'11; Random123 library): rounds of two 32x32->64 multiplies with the
constants below and a Weyl key schedule (ten rounds in Philox4x32-10).  The reference obtains its random bits from
Triton's ``tl.randint(seed, offset)`` (src/triton_kernels/fuse_kernel.py:30,
src/triton_kernels/stochastic_rounding_kernel.py:22), which is the same generator with
counter=(offset,0,0,0) and key=(seed,0), keeping only the first output word.  No
reference test pins that bit stream, so the CUDA library defines its own keying
(see ``sr_bits16``); this file is what the GPU stream is checked against.

Known-answer vectors from the Random123 distribution (kat_vectors, philox4x32 10) are
checked in tests/test_oracle_philox.py.
"""
import numpy as np

_M0 = np.uint64(0xD2511F53)
_M1 = np.uint64(0xCD9E8D57)
_W0 = np.uint64(0x9E3779B9)
_W1 = np.uint64(0xBB67AE85)
_MASK = np.uint64(0xFFFFFFFF)
_SH = np.uint64(32)


SR_ROUNDS = 7      # rounds of the CUDA library's own stochastic-rounding stream (csrc/numerics.cuh: kSrRounds)


def philox4x32(c0, c1, c2, c3, k0, k1, rounds=10):
    """Vectorised Philox4x32 with `rounds` rounds (10 = Philox4x32-10).  All arguments are broadcastable
    uint32 arrays (or ints).

    Returns four uint32 arrays.
    """
    c0, c1, c2, c3, k0, k1 = np.broadcast_arrays(
        *[np.asarray(v, dtype=np.uint64) & _MASK for v in (c0, c1, c2, c3, k0, k1)])
    c0 = c0.copy(); c1 = c1.copy(); c2 = c2.copy(); c3 = c3.copy()
    k0 = k0.copy(); k1 = k1.copy()
    for _ in range(rounds):
        p0 = _M0 * c0                       # 64-bit products; operands < 2^32 so no overflow
        p1 = _M1 * c2
        hi0, lo0 = p0 >> _SH, p0 & _MASK
        hi1, lo1 = p1 >> _SH, p1 & _MASK
        n0 = (hi1 ^ c1 ^ k0) & _MASK
        n2 = (hi0 ^ c3 ^ k1) & _MASK
        c0, c1, c2, c3 = n0, lo1, n2, lo0
        k0 = (k0 + _W0) & _MASK
        k1 = (k1 + _W1) & _MASK
    return (c0.astype(np.uint32), c1.astype(np.uint32),
            c2.astype(np.uint32), c3.astype(np.uint32))


def philox4x32_10(c0, c1, c2, c3, k0, k1):
    """Philox4x32-10, the generator Triton's tl.randint is built on."""
    return philox4x32(c0, c1, c2, c3, k0, k1, 10)


def sr_bits16(elem_index, seed, step):
    """16 random bits per weight element, as the CUDA update kernel draws them.

    Keying (defined by this build, not by the reference): one call of Philox4x32 stopped after
    SR_ROUNDS = 7 rounds (same round function and key schedule as Philox4x32-10) serves eight
    consecutive elements of a weight row.  counter = (q_lo, q_hi, step_lo, step_hi) with
    q = elem_index // 8, key = (seed_lo, seed_hi).  Element j = elem_index % 8 takes the
    16-bit half (j & 1) of output word (j >> 1).  ``elem_index`` is the GLOBAL flat index
    label_row * d + column, so the stream does not depend on chunking or on how label
    rows are sharded across GPUs.
    """
    e = np.asarray(elem_index, dtype=np.uint64)
    q = e >> np.uint64(3)
    j = (e & np.uint64(7)).astype(np.int64)
    seed = np.uint64(seed); step = np.uint64(step)
    x = philox4x32(q & _MASK, q >> _SH, step & _MASK, step >> _SH, seed & _MASK, seed >> _SH, SR_ROUNDS)
    words = np.stack(x, axis=0)                                  # [4, ...]
    w = np.take_along_axis(words, (j >> 1)[None, ...], axis=0)[0]
    return ((w >> ((j & 1) * 16).astype(np.uint32)) & np.uint32(0xFFFF)).astype(np.uint32)


def triton_randint(seed, offsets):
    """``tl.randint(seed, offsets)`` of Triton (third-party dependency of the reference, pinned
    indirectly by torch==2.6.0 -> triton 3.2.0; same definition in triton 3.6.0,
    triton/language/random.py): Philox4x32-10 with counter = (offset, 0, 0, 0) for 32-bit offsets
    (negative int32 offsets are bit-cast), key = (seed & 0xffffffff, seed >> 32), first output word.
    This is the stream behind fuse_kernel.py:12,30,40 and stochastic_rounding_kernel.py:12,22.
    Pinned by tests/golden/gpu_sr_helpers.npz (outputs of the reference's own launcher on a B200)."""
    off = np.asarray(offsets).astype(np.int64) & 0xFFFFFFFF
    seed = int(seed) & (2 ** 64 - 1)
    return philox4x32_10(off.astype(np.uint64), 0, 0, 0, seed & 0xFFFFFFFF, seed >> 32)[0]
