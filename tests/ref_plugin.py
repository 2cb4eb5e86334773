"""pytest plugin that runs a tsfast test session with the B200 backend installed.

Loaded with ``-p ref_plugin`` (this folder on ``PYTHONPATH``) when tsfast's own, unmodified test
files are collected from the reference copy: ``tsfast_b200.install()`` swaps the B200 modules into
tsfast's dispatch registries before collection, so every test that asks for the ``"triton"`` family
or runs under ``"auto"`` on CUDA exercises this repository's kernels.  At the end of the session
the number of launches each B200 module saw and the outcome counts are written as JSON to
``$B200_DROPIN_REPORT`` (if set), so the caller can check that the kernels, not tsfast's own, ran.
"""

import json
import os

_counts = {"passed": 0, "failed": 0, "skipped": 0, "failures": []}


def pytest_configure(config):
    import tsfast_b200

    config._b200_slots = tsfast_b200.install()


# fixtures of tsfast's conftest that open its dataset files; tests that ask for one train a Learner on
# recorded data, which is outside the scan path (and the files are not part of the reference copy)
_DATA_FIXTURES = {"wh_path", "pinn_var_ic_path", "hdf_files", "dls_simulation", "dls_short", "dls_prediction", "pinn_path",
                  "orientation_path", "dls_pinn"}


def pytest_collection_modifyitems(config, items):
    import pytest

    for item in items:
        if _DATA_FIXTURES & set(getattr(item, "fixturenames", ())):
            item.add_marker(pytest.mark.skip(reason="needs tsfast's dataset files (not on the scan path)"))


def pytest_runtest_logreport(report):
    if report.when == "call" or (report.when == "setup" and report.outcome != "passed"):
        _counts[report.outcome] = _counts.get(report.outcome, 0) + 1
        if report.outcome == "failed":
            _counts["failures"].append(report.nodeid)


def pytest_sessionfinish(session, exitstatus):
    import tsfast_b200
    from tsfast_b200 import allpole_b200, conv_b200, mamba_b200
    from tsfast_b200.scan_backends import diagonal_b200, selective_b200

    path = os.environ.get("B200_DROPIN_REPORT")
    if path:
        report = dict(_counts, exitstatus=int(exitstatus), slots=session.config._b200_slots,
                      launches={"scan.diagonal": diagonal_b200.calls, "scan.selective": selective_b200.calls,
                                "mamba.ssm": mamba_b200.calls, "mamba.conv": conv_b200.calls,
                                "dynonet.allpole": allpole_b200.calls})
        with open(path, "w") as f:
            json.dump(report, f, indent=1)
    tsfast_b200.uninstall()
