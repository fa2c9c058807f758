"""Makes the repository root importable when the scripts run with PYTHONPATH=helix_b200/scripts,
the way the reference's README runs them with PYTHONPATH=scripts."""
import os
import sys

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)
