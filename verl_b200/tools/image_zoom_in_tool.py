"""Image zoom-in tool (verl/tools/image_zoom_in_tool.py): the model asks for a crop ``bbox_2d = [x1, y1, x2, y2]`` of
the image attached to the trajectory and gets the (up-scaled) crop back as an image response. Boxes are clamped to
the image, and boxes smaller than ``min_size`` pixels are grown around their centre, as in the reference."""

from __future__ import annotations

from typing import Any, Optional
from uuid import uuid4

from .base_tool import BaseTool
from .schemas import OpenAIFunctionToolSchema, ToolResponse


class ImageZoomInTool(BaseTool):
    MIN_DIMENSION = 28

    def __init__(self, config: dict, tool_schema: OpenAIFunctionToolSchema):
        super().__init__(config, tool_schema)
        self._instances: dict[str, dict] = {}

    async def create(self, instance_id: Optional[str] = None, **kwargs):
        instance_id = instance_id or str(uuid4())
        ck = kwargs.get("create_kwargs") or kwargs
        image = ck.get("image")
        if image is None:
            raise ValueError("ImageZoomInTool needs 'image' in create_kwargs")
        self._instances[instance_id] = {"image": image}
        return instance_id, ToolResponse()

    def _valid_box(self, box, width: int, height: int):
        if not (isinstance(box, (list, tuple)) and len(box) == 4):
            return None
        x1, y1, x2, y2 = (float(v) for v in box)
        x1, y1, x2, y2 = max(0.0, x1), max(0.0, y1), min(float(width), x2), min(float(height), y2)
        if x2 <= x1 or y2 <= y1:
            return None
        m = self.MIN_DIMENSION
        if x2 - x1 < m or y2 - y1 < m:  # grow tiny boxes around their centre
            cx, cy = (x1 + x2) / 2, (y1 + y2) / 2
            w, h = max(x2 - x1, m), max(y2 - y1, m)
            x1, x2 = max(0.0, cx - w / 2), min(float(width), cx + w / 2)
            y1, y2 = max(0.0, cy - h / 2), min(float(height), cy + h / 2)
            if x2 - x1 < m or y2 - y1 < m:
                return None
        return int(x1), int(y1), int(round(x2)), int(round(y2))

    async def execute(self, instance_id: str, parameters: dict[str, Any], **kwargs):
        image = self._instances[instance_id]["image"]
        label = parameters.get("label", "")
        width, height = image.size if hasattr(image, "crop") else (image.shape[1], image.shape[0])  # PIL or HxWxC array
        box = self._valid_box(parameters.get("bbox_2d"), width, height)
        if box is None:
            return ToolResponse(text=f"Error: bbox_2d {parameters.get('bbox_2d')} is not a usable box inside the "
                                     f"{width}x{height} image"), -0.05, {"success": False}
        if hasattr(image, "crop"):
            crop = image.crop(box)
        else:
            crop = image[box[1] : box[3], box[0] : box[2]]
        text = f"Zoomed in on the image to the region {list(box)}" + (f" with label {label}." if label else ".")
        return ToolResponse(image=[crop], text=text), 0.0, {"success": True}

    async def release(self, instance_id: str, **kwargs) -> None:
        self._instances.pop(instance_id, None)
