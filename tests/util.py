"""Comparison rules of the parity tests: the shared checker in oracle/parity.py."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle.parity import (assert_parity, check_rows, compare, exact_rows_f64, rows_slack,  # noqa: E402,F401
                           summation_slack, summation_slack_grouped, _ordered, _ulp16)
