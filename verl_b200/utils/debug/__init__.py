"""Debug helpers: rollout-vs-trainer probability metrics, memory logging, trajectory tracking."""

from .metrics import calculate_debug_metrics, calculate_token_list_diff

__all__ = ["calculate_debug_metrics", "calculate_token_list_diff"]
