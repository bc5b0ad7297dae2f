"""The C-ABI library loads without a GPU and exports every symbol include/cafe_b200.h declares."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "cafe_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"^\s*(?:const\s+)?[A-Za-z_][\w\s\*]*?\b([A-Za-z_]\w*)\s*\([^;{]*\)\s*;", text, flags=re.M)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    from cafe_b200 import _lib, build
    build.build()
    lib = ctypes.CDLL(str(_lib.SO_PATH))
    names = declared_symbols()
    assert len(names) >= 30, names
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    # the Python binding table covers the same set
    assert sorted(_lib.SIGNATURES) == names


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from cafe_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "SO_PATH", tmp_path / "nope.so")
    import pytest
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.load()


def test_sizing_matches_reference_formulas():
    from cafe_b200 import sizing, synthetic
    # hot rows for the named configurations (reference: dlrm_s_pytorch.py:1239-1240)
    assert sizing.hot_rows(sum(synthetic.KAGGLE_CARDS), 0.001, 0.3, 16) == 13505
    assert sizing.hot_rows(sum(synthetic.MICRO_CARDS), 0.001, 0.3, 128) == 665600
    assert sizing.hot_rows(sum(synthetic.TERABYTE_CARDS), 0.001, 0.3, 128) == 120171
    assert sizing.hot_rows(sum(synthetic.TERABYTE_CARDS), 0.0001, 0.2, 128) == 13733
    assert sizing.hot_rows(sum(synthetic.AVAZU_CARDS), 0.1, 0.7, 16) == 161986
    assert sizing.hash_rows(40_000_000, 0.001, 0.3) == 12001
    assert sum(sizing.is_sketch_field(n, 0.1) for n in synthetic.AVAZU_CARDS) == 9
    assert sizing.field_offsets([3, 5, 7]) == [0, 3, 8]
