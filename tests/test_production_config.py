"""`.ako4x/production.toml`: the production-gate configuration the reference's supervisor loads
(ako4x/production_config.py:15-27 and load_production_config of the reference). The rules of that
loader are restated here so that the file is checked wherever the tests run; where a reference
checkout is mounted its own loader is used as well."""
import sys
import tomllib
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
CONFIG = ROOT / ".ako4x" / "production.toml"
REQUIRED_GATES = {"correctness", "numerical", "api-lifetime", "stream", "concurrency", "process-state",
                  "benchmark-integrity", "training-integration", "clean-deployment", "fallback", "reviewability"}


def test_config_follows_the_loader_rules():
    data = tomllib.loads(CONFIG.read_text())
    assert data["version"] == 1
    root = (CONFIG.parent / data["project"]["root"]).resolve()
    assert root == ROOT
    candidate = (root / data["project"]["candidate"]).resolve()
    assert candidate.exists()
    protected = [(root / p).resolve() for p in data["integrity"]["protected"]]
    assert protected
    for p in protected:
        assert p.exists() and p.is_relative_to(root)
        assert not (candidate == p or candidate.is_relative_to(p) or p.is_relative_to(candidate))
    for name in ("baseline", "benchmark"):
        assert data["commands"][name]["command"] and data["commands"][name]["timeout"] > 0
    for prof in ("ncu", "nsys"):
        raw = data["profilers"][prof]
        assert Path(raw["executable"]).name == prof
        for stage in ("smoke", "baseline", "candidate"):
            st = raw[stage]
            assert prof in {Path(tok).name for tok in st["command"]}
            assert st["parse"]["command"]
            assert Path(st["report"]).suffix == f".{prof}-rep"
            if prof == "ncu":   # this pool's rule: never let ncu lock the clocks
                cmd = st["command"]
                assert "--clock-control" in cmd and cmd[cmd.index("--clock-control") + 1] == "none"
    gates = {g["name"]: g for g in data["gate"]}
    assert set(gates) == REQUIRED_GATES and len(data["gate"]) == len(REQUIRED_GATES)
    for g in gates.values():
        assert g["command"]
        # every test file a gate names exists
        for tok in g["command"]:
            if tok.startswith("tests/"):
                assert (ROOT / tok).exists(), tok


def test_reference_loader_accepts_the_config():
    ref = Path("/root/reference")
    if not (ref / "ako4x" / "production_config.py").exists():
        pytest.skip("no reference checkout here")
    sys.path.insert(0, str(ref))
    try:
        from ako4x.production_config import load_production_config
        cfg = load_production_config(CONFIG)
    finally:
        sys.path.remove(str(ref))
    assert len(cfg.gates) == 11 and [p.name for p in cfg.profilers] == ["ncu", "nsys"]
