"""pytest configuration: registers the ``gpu`` marker and makes the in-tree package importable.

The package directory is ``2by4-pretrain_b200`` (not an importable name); the
drop-in Python package it holds is called ``sparse``, like the reference's.
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "2by4-pretrain_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
