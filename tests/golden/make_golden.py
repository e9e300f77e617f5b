"""Generate the golden fixtures in this folder by IMPORTING THE REFERENCE'S PYTHON.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

What the reference can execute without a GPU is exactly its host-side logic:
``recommend_coefficients``, ``RoutingMixin.router``, ``_adjust_lr`` and the
momentum / weight-decay / update arithmetic of ``muon_step`` (with its device
check patched out and a stand-in for the Newton-Schulz call, which needs CUDA).
The fixtures pin those against the reference's own code.  The stand-in NS is
``y = 3 * x`` rounded to x's dtype, so that the update path is exercised with a
known function.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent


def stand_in_ns(x, coeffs=None, eps=1e-7, deterministic=True, precision=None):
    return (x.float() * 3.0).to(x.dtype)


def main(reference_root: str) -> None:
    sys.path.insert(0, str(Path(reference_root) / "src"))
    import i8muon
    from i8muon import _optimizer as ref_opt

    # ---- coefficients
    coeffs = {}
    for method in ("int8_safe", "polar_express"):
        for iters in (1, 3, 5, 6, 7, 8, 10):
            try:
                coeffs[f"{method}:{iters}"] = i8muon.recommend_coefficients(iters, method=method)
            except ValueError as e:
                coeffs[f"{method}:{iters}"] = {"error": str(e)}
    shipped = json.loads((Path(reference_root) / "coefficients" / "int8_safe.json").read_text())
    coeffs["shipped_int8_safe_json"] = shipped["coefficients"]

    # ---- router
    class Probe(ref_opt.RoutingMixin):
        def _mk(name):
            def f(self, *a, **k):
                raise NotImplementedError
            f.__name__ = name
            return f
        _regular_prec = _mk("_regular_prec")
        _gram_prec = _mk("_gram_prec")
        _regular_i8 = _mk("_regular_i8")
        _regular_bq = _mk("_regular_bq")

    probe = Probe()
    routes = []
    shapes = [(768, 3072), (1024, 8192), (4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336),
              (2048, 8192), (128, 128), (32, 128), (1000, 1000), (1024, 1024), (1023, 1025), (64, 4096)]
    for M, N in shapes:
        for precision in ("auto", "int8", "i8", "int8_bq", "fp8", "fp8_bq", "float16", "bf16", "float32", "half"):
            for use_gram in (True, False):
                for thr in (5.0, 4.0):
                    fn, compute = probe.router(M, N, precision, use_gram, thr)
                    routes.append([M, N, precision, use_gram, thr, fn.__name__, compute])

    # ---- adjust_lr
    adjust = []
    for shape in [(768, 3072), (3072, 768), (4096, 4096), (3, 14336, 4096), (2048, 8192)]:
        for name in ("spectral", "original", "match_rms_adamw", "none", None):
            adjust.append([list(shape), name, ref_opt._adjust_lr(0.02, name, torch.Size(shape))])

    # ---- muon_step arithmetic with a stand-in NS
    ref_opt._validate_ns_device = lambda *a, **k: None

    class Engine:
        fp16_first = True
        tiles = {}

        def router(self, M, N, precision, use_gram, thr):
            return stand_in_ns, "float16"

    cases = []
    tensors = {}
    gen = torch.Generator().manual_seed(1234)
    index = 0
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        for momentum in ((0.95, 0.95), (0.9,), (0.3, 0.8)):
            for mode, wd in (("base_lr", 0.01), ("adjusted_lr", 0.01), ("absolute", 0.001), ("base_lr", 0.0)):
                for adjust_fn in ("spectral", "match_rms_adamw"):
                    shape = (2, 8, 24) if index % 2 else (17, 9)
                    p = (torch.randn(shape, generator=gen) * 0.02).to(dtype)
                    b = (torch.randn(shape, generator=gen) * 1e-3).to(dtype)
                    grads = [(torch.randn(shape, generator=gen) * 1e-3).to(dtype) for _ in range(2)]
                    key = f"case{index}"
                    tensors[key + ".param0"] = p.clone()
                    tensors[key + ".buf0"] = b.clone()
                    for s, g in enumerate(grads):
                        tensors[f"{key}.grad{s}"] = g.clone()
                        ref_opt.muon_step([p], [g], [b], lr=0.02, weight_decay=wd, momentum=momentum,
                                          ns_coefficients=None, eps=1e-7, adjust_lr_fn=adjust_fn,
                                          ns_engine=Engine(), precision="float16", use_gram=False,
                                          weight_decay_mode=mode)
                        tensors[f"{key}.param{s + 1}"] = p.clone()
                        tensors[f"{key}.buf{s + 1}"] = b.clone()
                    cases.append(dict(key=key, dtype=str(dtype), momentum=list(momentum), mode=mode, wd=wd,
                                      adjust=adjust_fn, shape=list(shape), lr=0.02))
                    index += 1

    (HERE / "reference_host_logic.json").write_text(json.dumps(
        dict(coefficients=coeffs, routes=routes, adjust_lr=adjust, muon_step_cases=cases), indent=1))
    torch.save(tensors, HERE / "reference_muon_step.pt")
    print("wrote", len(routes), "routes,", len(cases), "muon_step cases")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path of a checkout of the reference project>")
    main(sys.argv[1])
