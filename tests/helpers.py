"""Helpers of the parity tests: the oracle's view of a synthetic layer lives in oracle/layer_check.py."""
from oracle.layer_check import (error_metrics, np_u16, oracle_desc, oracle_experts, oracle_shared,  # noqa: F401
                                run_oracle)
