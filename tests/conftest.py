import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session", autouse=True)
def _built():
    """Builds the oracle here when it is missing; the product library must already exist."""
    so = os.path.join(ROOT, "oracle", "libfw_oracle.so")
    if not os.path.exists(so):
        env = dict(os.environ)
        env.pop("CC", None)
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle")], check=True, env=env)
    yield


# Lines a test wants in the record of a run that passes as well (pytest -q hides the output of
# passing tests): observed statistics of the distribution tests.
REPORT_LINES = []


def pytest_terminal_summary(terminalreporter):
    if REPORT_LINES:
        terminalreporter.write_sep("-", "observed statistics")
        for ln in REPORT_LINES:
            terminalreporter.write_line(ln)
