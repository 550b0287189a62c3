"""Shared pytest set-up: the `gpu` marker, the import path of the hyphenated
package directory, and small helpers used by several test files."""
import importlib
import os
import sys

import pytest

REPO_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO_ROOT not in sys.path:
    sys.path.insert(0, REPO_ROOT)

PACKAGE_NAME = "custom-tensorflow-compute-capability-sm-120_b200"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (compute capability 10.x) GPU")


@pytest.fixture(scope="session")
def pkg():
    return importlib.import_module(PACKAGE_NAME)


@pytest.fixture(scope="session")
def ops(pkg):
    return pkg.sm120_ops


@pytest.fixture(scope="session")
def binding(pkg):
    return pkg._binding
