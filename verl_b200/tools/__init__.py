from .base_tool import BaseTool
from .schemas import OpenAIFunctionToolSchema, ToolResponse

__all__ = ["BaseTool", "OpenAIFunctionToolSchema", "ToolResponse"]
