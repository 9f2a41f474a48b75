"""OpenAI-style function-tool schemas and tool results (verl/tools/schemas.py)."""

from __future__ import annotations

import json
from typing import Any, Literal, Optional

from pydantic import BaseModel, Field


class OpenAIFunctionPropertySchema(BaseModel):
    type: str
    description: Optional[str] = None
    enum: Optional[list[str]] = None


class OpenAIFunctionParametersSchema(BaseModel):
    type: str = "object"
    properties: dict[str, OpenAIFunctionPropertySchema] = Field(default_factory=dict)
    required: list[str] = Field(default_factory=list)


class OpenAIFunctionSchema(BaseModel):
    name: str
    description: str = ""
    parameters: OpenAIFunctionParametersSchema = Field(default_factory=OpenAIFunctionParametersSchema)
    strict: bool = False


class OpenAIFunctionToolSchema(BaseModel):
    type: str = "function"
    function: OpenAIFunctionSchema


class OpenAIFunctionParsedSchema(BaseModel):
    name: str
    arguments: str


class OpenAIFunctionCallSchema(BaseModel):
    name: str
    arguments: dict[str, Any]

    @staticmethod
    def from_openai_function_parsed_schema(parsed: OpenAIFunctionParsedSchema):
        bad = False
        try:
            args = json.loads(parsed.arguments)
        except json.JSONDecodeError:
            args, bad = {}, True
        if not isinstance(args, dict):
            args, bad = {}, True
        return OpenAIFunctionCallSchema(name=parsed.name, arguments=args), bad


class OpenAIFunctionToolCall(BaseModel):
    id: str
    type: Literal["function"] = "function"
    function: OpenAIFunctionCallSchema


class ToolResponse(BaseModel):
    """What a tool returns to the conversation: text and / or images / videos."""

    text: Optional[str] = None
    image: Optional[list[Any]] = None
    video: Optional[list[Any]] = None

    def is_empty(self) -> bool:
        return not self.text and not self.image and not self.video

    def is_text_only(self) -> bool:
        return bool(self.text) and not self.image and not self.video
