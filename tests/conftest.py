import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
  sys.path.insert(0, ROOT)


def pytest_configure(config):
  config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
  if torch.cuda.is_available():
    return
  skip = pytest.mark.skip(reason="no CUDA device")
  for item in items:
    if "gpu" in item.keywords:
      item.add_marker(skip)


class Golden:
  """Read access to tests/golden/qmm_golden.npz (made by tests/golden/make_golden.py)."""

  def __init__(self):
    self._z = np.load(os.path.join(ROOT, "tests", "golden", "qmm_golden.npz"))

  def np(self, key):
    return self._z[key]

  def t(self, key, bf16=False):
    a = self._z[key]
    if bf16:
      assert a.dtype == np.uint16
      return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
    return torch.from_numpy(a.copy())


@pytest.fixture(scope="session")
def golden():
  return Golden()
