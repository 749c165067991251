import os
import sys

# the kernel-selection knobs (chop_set_tuning) are a test facility: the library ignores them unless the process opts in
os.environ.setdefault("CHOP_ENABLE_TUNING", "1")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
