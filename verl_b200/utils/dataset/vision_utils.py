"""Image / video pre-processing for multimodal prompts (verl/utils/dataset/vision_utils.py:22-103): decode to RGB and
resize so that both sides are multiples of ``2 * patch`` within the min/max pixel budget (the Qwen-VL "smart resize"
rule). Video decoding needs a decoder package that this image does not have; frames given as arrays are accepted."""

from __future__ import annotations

import math
from io import BytesIO

import numpy as np


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280):
    if max(height, width) / max(1, min(height, width)) > 200:
        raise ValueError("absolute aspect ratio must be smaller than 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h, w = math.floor(height / beta / factor) * factor, math.floor(width / beta / factor) * factor
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h, w = math.ceil(height * beta / factor) * factor, math.ceil(width * beta / factor) * factor
    return max(factor, h), max(factor, w)


def process_image(image, image_patch_size: int = 14):
    """``image``: PIL image, HxWxC array, or dict with ``bytes`` / ``image`` and optional ``min_pixels`` / ``max_pixels``."""
    from PIL import Image

    opts = {}
    if isinstance(image, dict):
        opts = image
        image = image.get("image", image.get("bytes"))
        if isinstance(image, (bytes, bytearray)):
            image = Image.open(BytesIO(image))
    if isinstance(image, np.ndarray):
        image = Image.fromarray(image)
    image = image.convert("RGB")
    factor = 2 * image_patch_size
    h, w = smart_resize(image.height, image.width, factor, opts.get("min_pixels", 4 * factor * factor),
                        opts.get("max_pixels", 16384 * factor * factor))
    return image if (h, w) == (image.height, image.width) else image.resize((w, h))


def process_video(video, image_patch_size: int = 14, nframes: int | None = None, fps: float | None = None, **kwargs):
    """``video``: dict with ``frames`` (list of images / arrays) or an array [T, H, W, C]; samples ``nframes`` evenly."""
    frames = video.get("frames") if isinstance(video, dict) else video
    if frames is None:
        raise NotImplementedError("decoding video files needs a video decoder package; pass decoded frames")
    frames = list(frames)
    if nframes and nframes < len(frames):
        idx = np.linspace(0, len(frames) - 1, nframes).round().astype(int)
        frames = [frames[i] for i in idx]
    return [process_image(f, image_patch_size) for f in frames]
