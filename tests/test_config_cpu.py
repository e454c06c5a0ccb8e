"""Every TPB_* environment variable that the sources read is in the registry, with its default."""
import os
import re
from pathlib import Path

import pytest

import tensorplay_b200 as tp


def test_registry_covers_the_knobs_the_sources_read(monkeypatch):
    root = Path(tp.__file__).parent
    read = set()
    for f in root.rglob("*.py"):
        if f.name == "config.py":
            continue
        for m in re.finditer(r"environ(?:\.get|\.setdefault|\[)\(?\s*[\"'](TPB_[A-Z0-9_]+)[\"']", f.read_text()):
            read.add(m.group(1))
    known = set(tp.config.flags())
    assert read <= known, f"not in the registry: {sorted(read - known)}"
    monkeypatch.delenv("TPB_COMM_TRANSPORT", raising=False)
    assert tp.config.get("TPB_COMM_TRANSPORT") == "ce" and not tp.config.flags()["TPB_COMM_TRANSPORT"].is_set
    monkeypatch.setenv("TPB_COMM_TRANSPORT", "sm")
    assert tp.config.get("TPB_COMM_TRANSPORT") == "sm" and "TPB_COMM_TRANSPORT" in tp.config.describe(only_set=True)
    monkeypatch.setenv("TPB_SYMM_CANARY", "1")
    assert tp.config.get_bool("TPB_SYMM_CANARY") and not tp.config.get_bool("TPB_DEBUG") or os.environ.get("TPB_DEBUG") == "1"
    with pytest.raises(KeyError):
        tp.config.get("TPB_NO_SUCH_KNOB")
    f = tp.config.register("TPB_TEST_ONLY_KNOB", "7", "a knob of a test")
    assert tp.config.get("TPB_TEST_ONLY_KNOB") == "7" and f.doc == "a knob of a test"
    with pytest.raises(ValueError):
        tp.config.register("TPB_TEST_ONLY_KNOB", "8", "a knob of a test")
