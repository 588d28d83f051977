"""Host side of the per-tensor scale bookkeeping: the initial scale and the keeper's decisions."""
import math

from elmo_b200.scale import ScaleKeeper, initial_scale


def test_initial_scale_puts_the_bound_between_16_and_32():
    for L in (1000, 131072, 670208, 8623872):
        bound = math.sqrt(6.0 / (768 + L))                      # Xavier-uniform bound of the FP8 class
        s = initial_scale(bound)
        assert 16 <= bound / s < 32 and math.log2(s) == int(math.log2(s))
    assert initial_scale(0.0) == 1.0


def _st(amax, zero=0.0, sub=0.0, sat=0.0):
    return {"amax_stored": amax, "frac_zero": zero, "frac_subnormal": sub, "frac_saturated": sat, "elements": 1000}


def test_keeper_decisions():
    k = ScaleKeeper(interval=10)
    assert k.decide(_st(448.0, sat=1e-3)) == 1                  # saturated values: make room
    assert k.decide(_st(240.0)) == 1                            # within a binade of the top
    assert k.decide(_st(0.0039, zero=0.3, sub=0.6)) == -1       # the reference's start: everything sub-normal
    assert k.decide(_st(4.0, zero=0.01, sub=0.05)) == 0         # small but in the normal range
    assert k.decide(_st(32.0, zero=0.3, sub=0.3)) == 0          # lifting would not fit the large ones safely


class _FakeHandle:
    def __init__(self, stats):
        self.stats, self.calls, self.w_scale = stats, [], 1.0

    def weight_stats(self):
        return dict(self.stats)

    def rescale(self, shift, **kw):
        self.calls.append((shift, kw))
        self.w_scale *= 2.0 ** shift


def test_keeper_runs_only_on_its_interval_and_logs():
    h = _FakeHandle(_st(0.0039, zero=0.3, sub=0.6))
    k = ScaleKeeper(interval=4)
    applied = [k.maybe_update(h, it, seed=7) for it in range(1, 10)]
    assert applied == [0, 0, 0, -1, 0, 0, 0, -1, 0]
    assert [c[0] for c in h.calls] == [-1, -1] and h.w_scale == 0.25
    assert all(c[1]["stochastic"] and c[1]["seed"] == 7 for c in h.calls)
    assert [e["iteration"] for e in k.history] == [4, 8]
    assert ScaleKeeper(interval=0).maybe_update(h, 4, seed=7) == 0 and len(h.calls) == 2
