import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
if os.path.dirname(os.path.abspath(__file__)) not in sys.path:
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "slow: takes tens of seconds (a model of real width and vocabulary)")


def pytest_collection_modifyitems(config, items):
    # the file that must run last keeps its place even when files are given in another order
    items.sort(key=lambda it: (1 if "test_zz_" in it.nodeid else 0))
