"""The C-ABI library loads and exports every symbol include/hses.h declares
(no compute call is made, so this runs without a GPU)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "hses.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hses_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    syms = declared_symbols()
    for must in ("hses_ctx_create", "hses_lora_factors", "hses_perturbed_linear", "hses_poisson_encode",
                 "hses_lif_scan", "hses_es_update", "hses_solver_step", "hses_convert_fitnesses"):
        assert must in syms


def test_library_exports_every_declared_symbol():
    from hyperscalees_b200 import _lib
    assert os.path.exists(_lib.LIB_PATH), "build the library first (python -m hyperscalees_b200._build)"
    lib = ctypes.CDLL(_lib.LIB_PATH)
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, missing
    assert sorted(_lib.EXPORTS) == declared_symbols()


def test_pure_host_entry_points_work_without_a_gpu(oracle):
    from hyperscalees_b200 import _lib
    L = _lib.load()
    assert L.hses_version() >= 1
    for key, te, tt in [(0x9E3779B97F4A7C15, 0, 0), (7, 3, 5), (2**64 - 1, -1, -7)]:
        assert int(L.hses_noise_seed(key, te, tt)) == oracle.noise_seed(key, te, tt)
    assert L.hses_es_update_workspace_bytes(128, 784, 4, 256) > 0
    assert L.hses_es_update_workspace_bytes(0, 784, 4, 256) == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from hyperscalees_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    try:
        _lib.load()
    except RuntimeError as e:
        assert "no CPU or PyTorch fallback" in str(e)
    else:
        raise AssertionError("loading a missing library must raise")
