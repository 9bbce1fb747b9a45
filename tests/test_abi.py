"""The C-ABI library loads and exports every symbol that include/*.h declares (no compute, runs without a GPU)."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _declared(header: Path):
    text = header.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(db2[khw]?_[A-Za-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    from daphne_b200 import lib
    names = []
    for h in sorted((ROOT / "include").glob("*.h")):
        names += _declared(h)
    assert len(names) > 40
    missing = [n for n in names if not hasattr(lib.lib, n)]
    assert not missing, f"declared in include/ but not exported: {missing}"


def test_python_binding_covers_the_header():
    from daphne_b200 import lib
    declared = set()
    for h in sorted((ROOT / "include").glob("*.h")):
        declared |= set(_declared(h))
    bound = set(lib.exported_symbols())
    assert bound <= declared, f"bound but not declared: {sorted(bound - declared)}"


def test_no_device_is_reported_as_an_error_not_a_fallback():
    from daphne_b200 import lib
    import daphne_b200.kernels as k
    if lib.device_count() == 0:
        try:
            k.Context(0)
        except k.Db2Error as e:
            assert "no CPU fallback" in str(e)
        else:
            raise AssertionError("creating a context without a device must fail")
