"""Measured parity figures of a test run, for the record.

When the environment variable ``LF_PARITY_REPORT`` names a file, every GPU parity test that calls
``record`` appends one JSON line (test name, case, measured relative L2 error, bound) to it.  The tests
assert their bounds either way; the file only keeps the measured values next to them."""
import json
import os


def record(test, case, error, bound, **extra):
    path = os.environ.get("LF_PARITY_REPORT")
    if not path:
        return
    line = {"test": test, "case": case, "rel_l2": float(error), "bound": float(bound)}
    line.update(extra)
    with open(path, "a") as f:
        f.write(json.dumps(line) + "\n")
