"""CPU: host-side logic of the call sites (routing, normalisation) against the oracle restatement."""
import numpy as np

from nve_b200.gpu_layer import RoutingConfig, normalize_importance


def test_routing_matches_oracle(orc, golden):
    scores = golden["r_scores"]
    norm = normalize_importance(list(scores))
    assert np.array_equal(np.array(norm), golden["r_norm"])
    for thr in (0.0, 0.3, 0.5, 0.7, 1.0):
        cfg = RoutingConfig(False, thr)
        for v in norm:
            assert cfg.use_w4a8(v) == orc.use_w4a8(v, thr, False)
    assert not any(RoutingConfig(True, 0.7).use_w4a8(v) for v in norm)


def test_routing_env_semantics():
    """src/gpu_layer.rs:1017-1025: NVE_NO_W4A8 set (any value) forces W4A16; threshold default 0.7; a value
    that does not parse falls back to the default."""
    assert RoutingConfig.from_env({}).threshold == 0.7 and not RoutingConfig.from_env({}).no_w4a8
    assert RoutingConfig.from_env({"NVE_NO_W4A8": ""}).no_w4a8
    assert RoutingConfig.from_env({"NVE_W4A8_THRESHOLD": "0.25"}).threshold == 0.25
    assert RoutingConfig.from_env({"NVE_W4A8_THRESHOLD": "abc"}).threshold == 0.7
    # importance 0.0 (no profile) selects W4A8, as the benchmark harness of the reference relies on
    assert RoutingConfig().use_w4a8(0.0)


def test_top_half_threshold_is_the_median(golden):
    """'Top 50% of the scores -> W4A16' is the predicate importance < threshold with the threshold at the
    16th largest normalised score."""
    norm = sorted(golden["r_norm"])
    thr = norm[len(norm) // 2]
    cfg = RoutingConfig(False, float(thr))
    routes = [cfg.use_w4a8(float(v)) for v in golden["r_norm"]]
    assert sum(routes) == len(routes) // 2


def test_degenerate_scores():
    assert normalize_importance([2.0, 2.0]) == [0.5, 0.5]
    assert normalize_importance([1.0, 3.0]) == [0.0, 1.0]
