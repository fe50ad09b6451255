"""pytest plugin used by tests/test_reference_suite.py: routes this package's compute entry points to the CPU oracle
(tests/fake_backend.py) before the reference's own test modules are collected, so that their CPU tensors run through this
package's host logic.  Test infrastructure only."""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (HERE, ROOT, os.path.join(ROOT, "moizmxfp4-public_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    import fake_backend
    fake_backend.install()
