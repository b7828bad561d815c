"""Shared pytest configuration: the `gpu` marker and import paths."""
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselect with -m 'not gpu'")


def pytest_sessionstart(session):
    """The tests bind the in-tree shared library; (re)build it when a source is newer."""
    from quantexperiments_b200.build import build
    build()
