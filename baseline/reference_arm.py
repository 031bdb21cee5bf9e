"""Reference arm of the benchmark: the unmodified reference engine on the same metric and config.

The reference has no installable package metadata (no ``setup.py`` / ``pyproject.toml``), so
``pip install --target baseline/_ref`` cannot produce ``baseline/_ref``; when that directory is absent
this arm reports why and exits 0.
"""
from __future__ import annotations

import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def run_reference_arm(a) -> None:
    ref = os.path.join(HERE, "_ref")
    if not os.path.isdir(os.path.join(ref, "opt_prime")):
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable":
                              "reference is not pip-installable (no setup.py/pyproject.toml) and imports "
                              "transformers.utils.fx, which transformers 5.5 does not ship"}), flush=True)
        return
    sys.path.insert(0, ref)
    raise SystemExit("reference arm present but not wired")
