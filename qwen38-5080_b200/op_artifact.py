"""Writer of the experiment-side artifact of an op check: ``op.json``, schema ``phase2-op/1``.

The reference judges a candidate kernel by an artifact that its op-check scripts write and its
validator reads (runner/experiment/op_artifact.py:14-22,136-230; rules in
runner/experiment/artifacts.py:922-1075): a candidate with a name and a numeric format, git
provenance, and per case a non-empty config, at least one gate, at least one gate whose name starts
with ``coverage:``, and at least one finite numeric metric; diagnostics are recorded but never
decide.  This module writes that contract for checks of this library, so that a run of it can be
handed to the reference's experiment tooling unchanged.  It computes nothing itself.
"""
from __future__ import annotations

import json
import math
import os
import subprocess
import sys
from pathlib import Path
from typing import Any

SCHEMA = "phase2-op/1"


def git_state(root: Path) -> dict[str, Any]:
    """commit / dirty / short status of the work tree at `root` (empty strings outside a repository)."""
    def run(*args: str) -> str:
        try:
            return subprocess.check_output(["git", "-C", str(root), *args], text=True, stderr=subprocess.DEVNULL).strip()
        except Exception:  # noqa: BLE001 - no git, or not a repository
            return ""
    status = [line for line in run("status", "--porcelain", "--untracked-files=no").splitlines() if line]
    return {"commit": run("rev-parse", "HEAD"), "dirty": bool(status), "status": status[:20], "untracked_source": []}


class OpCase:
    """Gates, diagnostics and metrics of one case."""

    def __init__(self, name: str, config: dict[str, Any]):
        self.name, self.config = name, dict(config)
        self.gates: list[dict[str, Any]] = []
        self.diagnostics: list[dict[str, Any]] = []
        self.metrics: dict[str, float] = {}

    @staticmethod
    def _item(name: str, ok: bool, detail: Any) -> dict[str, Any]:
        item: dict[str, Any] = {"name": name, "ok": bool(ok)}
        if detail is not None:
            item["detail"] = detail
        return item

    def gate(self, name: str, ok: bool, detail: Any = None) -> bool:
        self.gates.append(self._item(name, ok, detail))
        return bool(ok)

    def diag(self, name: str, ok: bool, detail: Any = None) -> None:
        self.diagnostics.append(self._item(name, ok, detail))

    def metric(self, name: str, value: float) -> None:
        if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(float(value)):
            raise TypeError(f"metric {name!r} must be a finite number")
        self.metrics[name] = float(value)

    @property
    def ok(self) -> bool:
        return bool(self.gates) and all(g["ok"] for g in self.gates)

    def to_dict(self) -> dict[str, Any]:
        return {"case": self.name, "config": self.config, "gates": self.gates, "diagnostics": self.diagnostics,
                "metrics": self.metrics}


class OpReport:
    """Collects cases, then writes ``{out_dir}/op.json`` atomically."""

    def __init__(self, out_dir, candidate_name: str, candidate_format: str, *, candidate_extra: dict[str, Any] | None = None,
                 argv: list[str] | None = None, root=None, environment: dict[str, Any] | None = None, steps: int | None = None):
        self.out_dir = Path(out_dir)
        self.root = Path(root) if root is not None else Path(__file__).resolve().parents[1]
        self.candidate_name, self.candidate_format = str(candidate_name), str(candidate_format)
        self.candidate_extra = dict(candidate_extra or {})
        self.argv = list(sys.argv if argv is None else argv)
        self.environment = dict(environment or {})
        self.steps = steps
        self.cases: list[OpCase] = []

    def case(self, name: str, **config: Any) -> OpCase:
        case = OpCase(str(name), config)
        self.cases.append(case)
        return case

    def finish(self) -> dict[str, Any]:
        if not self.cases:
            raise ValueError("no cases")
        if not self.candidate_name.strip() or not self.candidate_format.strip():
            raise ValueError("candidate name and format must be given (the format decides comparability)")
        if len({c.name for c in self.cases}) != len(self.cases):
            raise ValueError("case names must be unique")
        for case in self.cases:
            if not case.config:
                raise ValueError(f"case {case.name!r}: empty config")
            if not case.gates or not any(g["name"].startswith("coverage:") for g in case.gates):
                raise ValueError(f"case {case.name!r}: needs gates, one of them a coverage: gate")
            if not case.metrics:
                raise ValueError(f"case {case.name!r}: needs a numeric metric")
        state = git_state(self.root)
        payload = {
            "schema": SCHEMA,
            "candidate": {"name": self.candidate_name, "format": self.candidate_format, "commit": state["commit"],
                          **self.candidate_extra},
            "provenance": {"git": state, "argv": self.argv, "cwd": str(Path.cwd()), "environment": self.environment},
            "steps": self.steps,
            "summary": {"ok": all(c.ok for c in self.cases),
                        "cases": [{"case": c.name, "gates": len(c.gates), "gates_passed": sum(1 for g in c.gates if g["ok"]),
                                   "gates_failed": [g["name"] for g in c.gates if not g["ok"]]} for c in self.cases]},
            "cases": [c.to_dict() for c in self.cases],
        }
        self.out_dir.mkdir(parents=True, exist_ok=True)
        path = self.out_dir / "op.json"
        tmp = path.with_suffix(".json.tmp")
        tmp.write_text(json.dumps(payload, indent=2, ensure_ascii=False) + "\n", encoding="utf-8")
        os.replace(tmp, path)
        return payload


__all__ = ["SCHEMA", "OpCase", "OpReport", "git_state"]
