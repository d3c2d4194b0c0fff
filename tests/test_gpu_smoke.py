"""The driver's smoke hook must stay green: it is run on a fresh GPU box before the bench."""
import os
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_smoke_hook_runs():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if root not in sys.path:
        sys.path.insert(0, root)
    import __graft_entry__
    __graft_entry__.smoke()
