from .partial_single_turn_agent_loop import PartialSingleTurnAgentLoop  # noqa: F401
