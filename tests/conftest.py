import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
  config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


@pytest.fixture(autouse=True)
def _reset_parallel_state():
  from t5x_b200.parallel import state as pstate
  pstate.reset()
  yield
  pstate.reset()
