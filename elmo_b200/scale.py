"""Per-tensor FP8 scale bookkeeping for the e4m3 layer classes.

The reference keeps the weights at scale 1.0 (src/xmc_classifiers/chunked_fp8xmc_clf.py:101-102): Xavier
initialisation of a 670 K-label layer is bounded by 3e-3, below e4m3's smallest normal 2^-6, so the
stored weights start on {0, +-2^-9, +-2^-8} (:29-32).  Here real = stored * scale with a power-of-two
scale that is chosen at construction and followed while training:

* ``initial_scale(bound)``: the scale that puts the initialisation bound at a stored magnitude of 16..32 --
  four binades of head-room below 448, ten binades of normal numbers below.
* ``ScaleKeeper``: every ``interval`` steps one statistics pass over the weights (counts of zeros,
  sub-normal magnitudes, saturated values, the largest magnitude) decides:
    - values at +-448, or the largest magnitude within one binade of it  -> scale x 2 (make room);
    - the largest magnitude below 2^3 while more than ``low_frac`` of the weights sit below the normal
      range -> scale / 2 (lift them), as long as that cannot saturate anything.
  A change rewrites the stored weights by the inverse power of two (exact when growing; what falls off
  the grid when shrinking is rounded stochastically with the step's Philox stream), so the real weights
  are unchanged.  ``interval = 0`` switches the keeper off: the scale stays what it was constructed with.
"""
import math
from typing import List, Optional


def initial_scale(bound: float) -> float:
    """Power of two s with 16 <= bound / s < 32."""
    if not (bound > 0):
        return 1.0
    return 2.0 ** (math.floor(math.log2(bound)) - 4)


class ScaleKeeper:
    def __init__(self, interval: int = 0, *, sat_frac: float = 0.0, low_frac: float = 0.25, log: Optional[List] = None):
        self.interval = int(interval)
        self.sat_frac, self.low_frac = sat_frac, low_frac
        self.history = log if log is not None else []

    def decide(self, st: dict) -> int:
        """Shift (in powers of two) to apply to the scale for these statistics: +1, -1 or 0."""
        amax = st["amax_stored"]
        if st["frac_saturated"] > self.sat_frac or amax >= 224.0:
            return 1
        if amax < 8.0 and (st["frac_zero"] + st["frac_subnormal"]) > self.low_frac and st["elements"] > 0:
            return -1
        return 0

    def maybe_update(self, handle, iteration: int, seed: int) -> int:
        """Called once per train step by the layer; returns the shift applied (0 almost always)."""
        if self.interval <= 0 or iteration == 0 or iteration % self.interval != 0:
            return 0
        st = handle.weight_stats()
        shift = self.decide(st)
        if shift:
            # the rounding of a shrink draws from a stream of its own (step counter in the upper half)
            handle.rescale(shift, stochastic=True, seed=seed, step=(1 << 40) + iteration)
        self.history.append({"iteration": iteration, "shift": shift, **st})
        return shift
