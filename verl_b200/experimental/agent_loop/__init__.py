from .agent_loop import (AgentLoopBase, AgentLoopManager, AgentLoopMetrics, AgentLoopOutput, AgentLoopWorker,
                         AsyncLLMServerManager, register)
from .single_turn_agent_loop import SingleTurnAgentLoop
from .tool_agent_loop import ToolAgentLoop

__all__ = ["AgentLoopBase", "AgentLoopManager", "AgentLoopWorker", "AgentLoopOutput", "AgentLoopMetrics",
           "AsyncLLMServerManager", "register", "SingleTurnAgentLoop", "ToolAgentLoop"]
