"""verl/utils/debug/metrics.py names, implemented in the package ``__init__``."""

from . import calculate_debug_metrics, calculate_token_list_diff  # noqa: F401
