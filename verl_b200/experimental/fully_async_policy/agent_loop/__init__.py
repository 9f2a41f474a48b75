from .partial_single_turn_agent_loop import PartialSingleTurnAgentLoop  # noqa: F401
from .partial_tool_agent_loop import PartialToolAgentLoop  # noqa: F401
from .agent_loop import FullyAsyncAgentLoopManager, FullyAsyncAgentLoopWorker, FullyAsyncLLMServerManager  # noqa: F401
