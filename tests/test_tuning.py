"""Selection logic of the host-side kernel tuner (the reference's KernelFactory rules) with an
injected clock: no GPU involved."""
import pytest

from i8muon_b200.tuning import KernelFactory


def make(times, capturing=False):
    """A factory whose timer returns times[candidate][trial] and records the order of calls."""
    calls = []

    def timer(launch, candidate, trial):
        calls.append((trial, candidate))
        launch(candidate)
        return times[candidate][trial]
    return KernelFactory(True, timer=timer, capturing=lambda: capturing), calls


def test_autotune_off_returns_default_without_launching():
    launched = []
    factory = KernelFactory(False, timer=lambda *a: pytest.fail("timed"))
    assert factory.select("op", "k", (0, 1), 0, launched.append) == 0
    assert not factory.select_pipeline("fam", "k", launched.append)
    assert launched == []


def test_default_is_kept_unless_two_percent_faster():
    factory, _ = make({0: [1.00, 1.00, 1.00], 1: [0.985, 0.985, 0.985]})
    assert factory.select("op", "k", (0, 1), 0, lambda c: None) == 0      # 1.5 % is not enough
    factory, _ = make({0: [1.00, 1.00, 1.00], 1: [0.97, 0.97, 0.97]})
    assert factory.select("op", "k", (0, 1), 0, lambda c: None) == 1


def test_median_of_three_trials_in_rotated_order():
    # candidate 1 has one lucky outlier; its median is slower than the default
    factory, calls = make({0: [1.0, 1.0, 1.0], 1: [0.5, 1.1, 1.2], 2: [1.3, 1.3, 1.3]})
    assert factory.select("op", "k", (0, 1, 2), 0, lambda c: None) == 0
    assert calls == [(0, 0), (0, 1), (0, 2), (1, 1), (1, 2), (1, 0), (2, 2), (2, 0), (2, 1)]
    key = ("op", "k", (0, 1, 2))
    assert factory.timings[key] == {0: 1.0, 1: 1.1, 2: 1.3}


def test_result_is_cached_per_key():
    factory, calls = make({0: [1.0] * 3, 1: [0.5] * 3})
    assert factory.select("op", ("shape", 1), (0, 1), 0, lambda c: None) == 1
    n = len(calls)
    assert factory.select("op", ("shape", 1), (0, 1), 0, lambda c: None) == 1
    assert len(calls) == n
    factory.select("op", ("shape", 2), (0, 1), 0, lambda c: None)
    assert len(calls) == 2 * n


def test_tuning_inside_a_capture_is_refused_but_cached_choices_are_served():
    factory, _ = make({0: [1.0] * 3, 1: [0.5] * 3}, capturing=True)
    with pytest.raises(RuntimeError, match="Warm up"):
        factory.select("op", "k", (0, 1), 0, lambda c: None)
    factory.cache[("op", "k", (0, 1))] = 1
    assert factory.select("op", "k", (0, 1), 0, lambda c: None) == 1


def test_pipeline_needs_one_percent():
    factory, _ = make({False: [1.0] * 3, True: [0.995] * 3})
    assert factory.select_pipeline("bq", "k", lambda tuned: None) is False
    factory, _ = make({False: [1.0] * 3, True: [0.98] * 3})
    assert factory.select_pipeline("bq", "k", lambda tuned: None) is True


def test_default_must_be_a_candidate():
    factory, _ = make({0: [1.0] * 3, 1: [1.0] * 3})
    with pytest.raises(ValueError):
        factory.select("op", "k", (0, 1), 2, lambda c: None)
