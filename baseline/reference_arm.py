"""Reference arm of bench.py: runs the unmodified reference (installed under baseline/_ref) on the same metric.

When the reference cannot be imported, prints the ``unavailable`` JSON line and exits 0.
"""
from __future__ import annotations

import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def _unavailable(reason: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": reason}), flush=True)


def main(args) -> None:
    if not os.path.isdir(os.path.join(REF_DIR, "deep_ep")):
        _unavailable("reference not installed: its setup.py needs libfabric (rdma/fabric.h) and GDRCopy, absent from this image")
        return
    _unavailable("reference arm not wired yet")
