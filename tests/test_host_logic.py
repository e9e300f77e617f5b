"""Host-side logic against fixtures generated from the reference's own Python
(tests/golden/make_golden.py): coefficient tables, route selection, learning-rate
scaling, and the reference's error behaviour."""
import math

import pytest
import torch

from i8muon_b200 import CutlassNSInt8, Muon, recommend_coefficients
from i8muon_b200.routing import adjust_lr, matrix_spec, normalize_precision, select_route


def test_coefficients_match_reference(host_golden):
    for key, expected in host_golden["coefficients"].items():
        if key == "shipped_int8_safe_json":
            assert [list(r) for r in recommend_coefficients(5)] == expected
            continue
        method, iters = key.split(":")
        if isinstance(expected, dict):
            with pytest.raises(ValueError) as err:
                recommend_coefficients(int(iters), method=method)
            assert str(err.value) == expected["error"]
        else:
            got = recommend_coefficients(int(iters), method=method)
            assert [list(r) for r in got] == expected  # bit-identical python floats


def test_coefficients_argument_errors():
    with pytest.raises(TypeError):
        recommend_coefficients(True)
    with pytest.raises(ValueError):
        recommend_coefficients(5, method="nope")
    with pytest.raises(ValueError):
        recommend_coefficients(0, method="polar_express")
    assert len(recommend_coefficients(7)) == 7
    seven = recommend_coefficients(7)
    assert seven[2] == seven[3] == seven[4]


def test_routes_match_reference(host_golden):
    engine = CutlassNSInt8()
    for M, N, precision, use_gram, thr, name, compute in host_golden["routes"]:
        assert select_route(M, N, precision, use_gram, thr) == (name, compute)
        fn, got_compute = engine.router(M, N, precision, use_gram, thr)
        assert fn.__name__ == name and got_compute == compute


def test_route_errors():
    with pytest.raises(ValueError):
        select_route(0, 4, "auto", True, 5.0)
    with pytest.raises(ValueError):
        normalize_precision("int4")
    with pytest.raises(ValueError):
        normalize_precision(8)


def test_adjust_lr_matches_reference(host_golden):
    for shape, name, expected in host_golden["adjust_lr"]:
        assert adjust_lr(0.02, name, torch.Size(shape)) == expected
    assert adjust_lr(0.5, lambda lr, a, b: lr * a / b, (4, 8)) == 0.25


def test_matrix_spec_rejects_cpu_and_bad_dtypes():
    with pytest.raises(ValueError):
        matrix_spec((4, 4), torch.float32, torch.device("cpu"), "float16")


def test_engine_tiles_validation():
    CutlassNSInt8(tiles={"aat": 4, "square": 0})
    with pytest.raises(ValueError):
        CutlassNSInt8(tiles={"gram": 1})
    with pytest.raises(ValueError):
        CutlassNSInt8(tiles={"aat": 7})


# ------------------------------------------------------------------ optimizer surface on CPU
def _params():
    return [torch.nn.Parameter(torch.randn(8, 16)), torch.nn.Parameter(torch.randn(2, 4, 6))]


def test_muon_constructs_and_validates():
    opt = Muon(_params(), lr=0.02, weight_decay=0.1, ns_steps=6)
    group = opt.param_groups[0]
    assert len(group["ns_coefficients"]) == 6
    assert group["momentum"] == (0.95, 0.95) and group["precision"] == "auto"
    assert group["weight_decay_mode"] == "base_lr"
    for bad in (dict(weight_decay=-1.0), dict(eps=-1.0), dict(momentum=(0.1, 0.2, 0.3)),
                dict(adjust_lr_fn="bogus"), dict(precision="int3"), dict(weight_decay_mode="x"),
                dict(ns_coefficients=[]), dict(ns_coefficients=[(1, 2)])):
        with pytest.raises(ValueError):
            Muon(_params(), **bad)
    with pytest.raises(ValueError):
        Muon([torch.nn.Parameter(torch.randn(8))])
    with pytest.raises(ValueError):
        Muon(_params(), ns_steps=3)
    Muon(_params(), momentum=0.9)  # scalar momentum


def test_muon_scalar_optimizer_plumbing():
    matrices = _params()
    vectors = [torch.nn.Parameter(torch.randn(8))]
    aux = torch.optim.AdamW(vectors, lr=1e-3)
    opt = Muon(matrices, scalar_optimizer=aux)
    assert len(opt.param_groups) == 2 and opt.param_groups[1] is aux.param_groups[0]
    state = opt.state_dict()
    assert len(state["param_groups"]) == 1  # Muon state only
    assert set(state["param_groups"][0]) >= {"lr", "weight_decay", "weight_decay_mode", "momentum",
                                            "ns_coefficients", "eps", "adjust_lr_fn", "deterministic",
                                            "use_gram", "precision", "params"}
    with pytest.raises(ValueError):
        Muon(matrices, scalar_optimizer=torch.optim.AdamW(matrices[:1]))
    with pytest.raises(ValueError):
        opt.add_param_group({"params": vectors})  # 1-D parameter
    extra = torch.nn.Parameter(torch.randn(4, 4))
    opt.add_param_group({"params": [extra], "lr": 0.5})
    assert len(opt.param_groups) == 3 and opt.param_groups[1]["lr"] == 0.5
    with pytest.raises(TypeError):
        opt.add_param_group({"params": {torch.nn.Parameter(torch.randn(4, 4))}})


def test_muon_state_dict_round_trip_and_legacy_default():
    opt = Muon(_params(), weight_decay_mode="absolute")
    state = opt.state_dict()
    opt2 = Muon(_params())
    opt2.load_state_dict(state)
    assert opt2.param_groups[0]["weight_decay_mode"] == "absolute"
    for group in state["param_groups"]:
        del group["weight_decay_mode"]  # a checkpoint that predates the option
    opt3 = Muon(_params())
    opt3.load_state_dict(state)
    assert opt3.param_groups[0]["weight_decay_mode"] == "adjusted_lr"


def test_cpu_step_is_refused():
    params = _params()
    for p in params:
        p.grad = torch.randn_like(p)
    with pytest.raises(ValueError, match="CUDA"):
        Muon(params).step()
