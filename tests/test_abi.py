"""CPU checks of the C-ABI boundary: the library builds, loads, exports every symbol
the header declares, and refuses to run without a device (no CPU fallback)."""
import ctypes as C
import re
from pathlib import Path

import pytest

import larql_b200
from larql_b200 import build as lqbuild

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    lqbuild.build()
    return larql_b200.load_library()


def test_header_symbols_match_exports(lib):
    header = (ROOT / "include" / "larql_cuda.h").read_text()
    declared = sorted(set(re.findall(r"LQ_API\s+[\w\s\*]+?\b(lq_\w+)\s*\(", header)))
    assert declared, "no LQ_API declarations found"
    assert sorted(larql_b200.EXPORTS) == declared
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_every_entry_point_cites_the_reference():
    header = (ROOT / "include" / "larql_cuda.h").read_text()
    # each declaration is preceded by a comment naming a reference file or saying it has no counterpart
    assert header.count("crates/") >= 15


def test_no_cpu_fallback_without_device(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    h = C.c_void_p()
    assert lib.lq_create(0, C.byref(h)) != 0 and not h.value
    with pytest.raises(larql_b200.BackendError):
        larql_b200.CudaBackend(0)


def test_product_does_not_import_the_oracle():
    for p in list((ROOT / "larql_b200").rglob("*.py")) + list((ROOT / "larql_b200").rglob("*.cu*")) + \
            list((ROOT / "larql_b200").rglob("*.h")) + list((ROOT / "include").glob("*.h")):
        text = p.read_text()
        assert "import oracle" not in text and "larql_oracle" not in text and "from oracle" not in text, p


REFERENCE = Path("/root/reference")


def _resolve(rel: str):
    for base in ("", "crates/larql-compute/src/", "crates/larql-compute/src/cpu/", "crates/larql-models/src/",
                 "crates/larql-models/src/quant/"):
        p = REFERENCE / (base + rel)
        if p.is_file():
            return p
    return None


@pytest.mark.skipif(not REFERENCE.is_dir(), reason="the reference checkout is not on this machine")
def test_header_citations_point_at_the_named_code():
    """Every `path.rs:a-b` in the header exists with that many lines, and where the comment names a trait
    method (`Trait::method (path:a-b)`), the cited range holds `fn method`."""
    header = (ROOT / "include" / "larql_cuda.h").read_text()
    flat = re.sub(r"\s*\n\s*\*\s*", " ", header)
    cites = re.findall(r"([\w\-/\.…]+\.rs):(\d+)(?:-(\d+))?", flat)
    assert len(cites) >= 30
    for rel, a, b in cites:
        if rel.startswith("…"):
            continue  # abbreviated continuation of a path given in full just before
        p = _resolve(rel)
        assert p is not None, f"cited file not found: {rel}"
        n_lines = len(p.read_text().splitlines())
        assert int(b or a) <= n_lines, f"{rel}:{a}-{b} is past the end of the file ({n_lines} lines)"
    named = re.findall(r"(?:QuantMatVec|MatMul|ComputeBackend)::(\w+)(?:\(_force\))?\s*\(([\w\-/\.]+\.rs):(\d+)-(\d+)", flat)
    assert len(named) >= 8
    for method, rel, a, b in named:
        p = _resolve(rel)
        assert p is not None, rel
        body = "\n".join(p.read_text().splitlines()[int(a) - 1:int(b)])
        assert re.search(rf"fn {method}\b", body), f"{rel}:{a}-{b} does not define fn {method}"
