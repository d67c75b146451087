"""The op.json writer (CPU) and the op check that uses it (GPU): the artifact must satisfy the rules the
reference's validator applies to a phase2-op/1 artifact (runner/experiment/artifacts.py:922-1075)."""
import importlib
import json
import math
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def validate(data: dict) -> None:
    """The validator's rules, restated."""
    assert data["schema"] == "phase2-op/1"
    cand = data["candidate"]
    assert cand["name"].strip() and cand["format"].strip()
    git = data["provenance"]["git"]
    assert "commit" in git and "dirty" in git and cand["commit"] == git["commit"]
    names = [c["case"] for c in data["cases"]]
    assert names and len(names) == len(set(names))
    assert [c["case"] for c in data["summary"]["cases"]] == names
    for c in data["cases"]:
        assert isinstance(c["config"], dict) and c["config"]
        assert c["gates"] and any(g["name"].startswith("coverage:") for g in c["gates"])
        assert c["metrics"] and all(isinstance(v, float) and math.isfinite(v) for v in c["metrics"].values())
    assert data["summary"]["ok"] == all(g["ok"] for c in data["cases"] for g in c["gates"])


def test_writer_contract(tmp_path):
    art = importlib.import_module("qwen38-5080_b200.op_artifact")
    rep = art.OpReport(tmp_path, "cand", "fp8-kv", candidate_extra={"backend": "cuda-sm100a"}, steps=4, argv=["x"])
    c = rep.case("one", depth=512)
    c.gate("coverage: shapes", True)
    c.gate("parity", False, 0.5)
    c.diag("note", True, "text")
    c.metric("us", 1.5)
    with pytest.raises(TypeError):
        c.metric("bad", float("nan"))
    data = rep.finish()
    validate(data)
    assert json.loads((tmp_path / "op.json").read_text()) == data
    assert data["summary"]["ok"] is False and data["summary"]["cases"][0]["gates_failed"] == ["parity"]
    assert data["candidate"]["backend"] == "cuda-sm100a" and data["steps"] == 4
    for broken in ("no-gate", "no-coverage", "no-metric", "no-config"):
        rep = art.OpReport(tmp_path, "cand", "fp8-kv")
        c = rep.case("x", **({} if broken == "no-config" else {"depth": 1}))
        if broken != "no-gate":
            c.gate("parity" if broken == "no-coverage" else "coverage: x", True)
        if broken != "no-metric":
            c.metric("us", 1.0)
        with pytest.raises(ValueError):
            rep.finish()


@pytest.mark.gpu
def test_op_check_writes_a_passing_artifact(tmp_path, cuda_device):
    res = subprocess.run([sys.executable, str(ROOT / "tests" / "op_check.py"), "--out", str(tmp_path), "--steps", "4"],
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    data = json.loads((tmp_path / "op.json").read_text())
    validate(data)
    assert data["summary"]["ok"] is True and len(data["cases"]) == 3
