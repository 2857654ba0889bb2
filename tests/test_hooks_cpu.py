"""hooks.install() re-points the reference package's names at this library (and uninstall() restores them),
exercised on a stand-in `semicat` package tree so that no reference checkout is needed."""
import importlib
import sys
import textwrap

import pytest

from semicat_b200 import functional, hooks


@pytest.fixture
def fake_semicat(tmp_path, monkeypatch):
    root = tmp_path / "semicat"
    (root / "jvp_utils").mkdir(parents=True)
    (root / "net").mkdir()
    for d in (root, root / "jvp_utils", root / "net"):
        (d / "__init__.py").write_text("")
    (root / "jvp_utils" / "functional.py").write_text(textwrap.dedent("""
        def sdpa_jvp(q, k, v):
            return "reference sdpa_jvp"
        def safe_sdpa_jvp(q, k, v):
            return "reference safe_sdpa_jvp"
    """))
    (root / "net" / "duo.py").write_text("from semicat.jvp_utils.functional import safe_sdpa_jvp\n")
    monkeypatch.syspath_prepend(str(tmp_path))
    for name in [m for m in sys.modules if m == "semicat" or m.startswith("semicat.")]:
        monkeypatch.delitem(sys.modules, name)
    yield
    hooks.uninstall()
    for name in [m for m in sys.modules if m == "semicat" or m.startswith("semicat.")]:
        sys.modules.pop(name, None)


def test_install_repoints_definitions_and_early_importers(fake_semicat):
    duo = importlib.import_module("semicat.net.duo")  # bound the reference name at import time
    assert duo.safe_sdpa_jvp(None, None, None) == "reference safe_sdpa_jvp"
    patched = hooks.install(strict=True)
    ref = importlib.import_module("semicat.jvp_utils.functional")
    assert "semicat.jvp_utils.functional" in patched and "semicat.net.duo" in patched
    assert ref.sdpa_jvp is functional.sdpa_jvp and ref.safe_sdpa_jvp is functional.safe_sdpa_jvp
    assert duo.safe_sdpa_jvp is functional.safe_sdpa_jvp
    hooks.uninstall()
    assert duo.safe_sdpa_jvp(None, None, None) == "reference safe_sdpa_jvp"
    assert ref.sdpa_jvp(None, None, None) == "reference sdpa_jvp"


def test_install_without_reference_is_a_noop_unless_strict(monkeypatch):
    for name in [m for m in sys.modules if m == "semicat" or m.startswith("semicat.")]:
        monkeypatch.delitem(sys.modules, name)
    monkeypatch.setattr(sys, "path", [p for p in sys.path if "reference" not in p])
    try:
        importlib.import_module("semicat")
        pytest.skip("a real semicat package is importable here")
    except ImportError:
        pass
    assert hooks.install() == []
    with pytest.raises(ImportError):
        hooks.install(strict=True)
