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


_CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
_CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def images_to_patches(images, patch_size: int = 14, merge_size: int = 2, temporal_patch_size: int = 2,
                      mean=_CLIP_MEAN, std=_CLIP_STD):
    """What the Qwen2-VL image processor produces for still images: ``pixel_values [sum(h * w), C * T * P * P]``
    (float32; every image resized by :func:`process_image`, normalised, repeated over the temporal patch, cut into
    patches in 2 x 2 merge-block order) and ``image_grid_thw [n_images, 3]`` with the grid in patches
    (transformers' ``Qwen2VLImageProcessor``; verl/utils/dataset/rl_dataset.py builds ``multi_modal_inputs`` from it)."""
    import torch

    pvs, grids = [], []
    for img in images:
        im = process_image(img, patch_size)
        x = torch.from_numpy(np.asarray(im, dtype=np.float32) / 255.0)            # [H, W, 3]
        x = (x - torch.tensor(mean)) / torch.tensor(std)
        x = x.permute(2, 0, 1)                                                    # [3, H, W]
        C, H, W = x.shape
        gh, gw = H // patch_size, W // patch_size
        x = x.unsqueeze(0).repeat(temporal_patch_size, 1, 1, 1)                    # [T, 3, H, W]
        m = merge_size
        x = x.reshape(temporal_patch_size, C, gh // m, m, patch_size, gw // m, m, patch_size)
        # -> (gh/m, gw/m, m, m) patch order, each patch flattened as (C, T, P, P)
        x = x.permute(2, 5, 3, 6, 1, 0, 4, 7).reshape(gh * gw, C * temporal_patch_size * patch_size * patch_size)
        pvs.append(x)
        grids.append([1, gh, gw])
    return torch.cat(pvs, 0), torch.tensor(grids, dtype=torch.long)


def videos_to_patches(videos, patch_size: int = 14, merge_size: int = 2, temporal_patch_size: int = 2,
                      mean=_CLIP_MEAN, std=_CLIP_STD):
    """Videos (each a list / array of frames ``[T, H, W, 3]``, or a dict with ``frames``) -> ``pixel_values_videos
    [sum(t * h * w), C * temporal_patch_size * P * P]`` and ``video_grid_thw [n_videos, 3]``: every frame resized as a
    still image is, ``temporal_patch_size`` consecutive frames share a patch (the last frame is repeated to fill the
    last one), patches in 2 x 2 merge-block order frame group by frame group (what transformers'
    ``Qwen2VLVideoProcessor`` produces; verl/utils/dataset/vision_utils.py ``process_video``)."""
    import torch

    pvs, grids = [], []
    for video in videos:
        frames = process_video(video, patch_size)
        xs = []
        for im in frames:
            x = torch.from_numpy(np.asarray(im, dtype=np.float32) / 255.0)
            xs.append(((x - torch.tensor(mean)) / torch.tensor(std)).permute(2, 0, 1))
        x = torch.stack(xs)                                                         # [T, 3, H, W]
        pad = (-x.shape[0]) % temporal_patch_size
        if pad:
            x = torch.cat([x, x[-1:].repeat(pad, 1, 1, 1)], 0)
        T, C, H, W = x.shape
        gt, gh, gw, m = T // temporal_patch_size, H // patch_size, W // patch_size, merge_size
        x = x.reshape(gt, temporal_patch_size, C, gh // m, m, patch_size, gw // m, m, patch_size)
        # -> (gt, gh/m, gw/m, m, m) patch order, each patch flattened as (C, T, P, P)
        x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8).reshape(gt * gh * gw, C * temporal_patch_size * patch_size * patch_size)
        pvs.append(x)
        grids.append([gt, gh, gw])
    return torch.cat(pvs, 0), torch.tensor(grids, dtype=torch.long)


def expand_image_placeholders(ids: list[int], grids, image_token_id: int, merge_size: int = 2,
                              vision_start_id: int | None = None, vision_end_id: int | None = None) -> list[int]:
    """Every image placeholder token of ``ids`` becomes ``t * h * w / merge^2`` copies (one per merged patch), image by
    image; a prompt without placeholders gets the images in front (between the vision start / end tokens if given)."""
    counts = [int(t) * int(h) * int(w) // (merge_size * merge_size) for t, h, w in (grids.tolist() if hasattr(grids, "tolist") else grids)]
    if image_token_id not in ids:
        head: list[int] = []
        for n in counts:
            head += ([vision_start_id] if vision_start_id is not None else []) + [image_token_id] * n + \
                    ([vision_end_id] if vision_end_id is not None else [])
        return head + list(ids)
    out, k = [], 0
    i = 0
    while i < len(ids):
        if ids[i] == image_token_id:
            j = i
            while j < len(ids) and ids[j] == image_token_id:
                j += 1
            if k >= len(counts):
                raise ValueError("more image placeholders in the prompt than images")
            out += [image_token_id] * counts[k]   # a run of placeholders stands for ONE image
            k += 1
            i = j
        else:
            out.append(ids[i])
            i += 1
    if k != len(counts):
        raise ValueError(f"{len(counts)} images but {k} image placeholders in the prompt")
    return out


class VLProcessor:
    """What a dataset needs from a vision-language model to build multimodal prompts: the placeholder token, the patch
    geometry and the multimodal RoPE rule (role of the ``AutoProcessor`` the reference passes to ``RLHFDataset``,
    verl/utils/dataset/rl_dataset.py)."""

    def __init__(self, image_token_id: int, patch_size: int = 14, merge_size: int = 2, temporal_patch_size: int = 2,
                 vision_start_id: int | None = None, vision_end_id: int | None = None, video_token_id: int | None = None):
        self.image_token_id, self.patch_size, self.merge_size = int(image_token_id), int(patch_size), int(merge_size)
        self.temporal_patch_size = int(temporal_patch_size)
        self.vision_start_id, self.vision_end_id = vision_start_id, vision_end_id
        self.video_token_id = None if video_token_id is None else int(video_token_id)

    @classmethod
    def from_model_config(cls, cfg):
        if not getattr(cfg, "is_vl", False):
            return None
        v = cfg.extra.get("vision_config") or {}
        return cls(cfg.image_token_id, v.get("patch_size", 14), v.get("spatial_merge_size", 2), v.get("temporal_patch_size", 2),
                   cfg.extra.get("vision_start_token_id"), cfg.extra.get("vision_end_token_id"), cfg.extra.get("video_token_id"))

    def __call__(self, prompt_ids: list[int], images=None, videos=None):
        """-> (prompt ids with expanded placeholders, multi_modal_inputs dict, mrope positions [3, L]). A video's
        placeholder run stands for the whole video (one token per merged patch of every frame group); its temporal RoPE
        position advances by one per frame group (the Qwen2-VL rule; the per-second scaling of Qwen2.5-VL and the
        timestamp text between the frames of Qwen3-VL prompts are not modelled)."""
        from ...models.vision import get_rope_index
        import torch

        ids, mm, grid, vgrid = list(prompt_ids), {}, None, None
        if videos is not None and len(videos):
            assert self.video_token_id is not None, "this model has no video placeholder token"
            pvv, vgrid = videos_to_patches(videos, self.patch_size, self.merge_size, self.temporal_patch_size)
            ids = expand_image_placeholders(ids, vgrid, self.video_token_id, self.merge_size, self.vision_start_id,
                                            self.vision_end_id)
            mm.update(pixel_values_videos=pvv, video_grid_thw=vgrid)
        if images is not None and len(images):
            pv, grid = images_to_patches(images, self.patch_size, self.merge_size, self.temporal_patch_size)
            ids = expand_image_placeholders(ids, grid, self.image_token_id, self.merge_size, self.vision_start_id,
                                            self.vision_end_id)
            mm.update(pixel_values=pv, image_grid_thw=grid)
        pos3, _ = get_rope_index(torch.tensor(ids), grid, self.image_token_id, self.merge_size, video_grid_thw=vgrid,
                                 video_token_id=self.video_token_id)
        return ids, mm, pos3


def vl_position_ids(input_ids, attention_mask, multi_modal_inputs, image_token_id: int, merge_size: int = 2,
                    video_token_id: int | None = None):
    """[B, 4, S] position ids of padded sequences: row 0 = text positions, rows 1..3 = multimodal RoPE (temporal,
    height, width) from the unpadded tokens of every row and its image grid (verl/utils/dataset/rl_dataset.py and
    verl/models/transformers/qwen2_vl.py ``get_rope_index``)."""
    import torch

    from ...models.vision import get_rope_index

    B, S = input_ids.shape
    out = torch.zeros(B, 4, S, dtype=torch.long)
    text = (attention_mask.cumsum(-1) - 1).clamp(min=0)
    out[:, 0] = text
    for b in range(B):
        m = attention_mask[b].bool()
        mm = multi_modal_inputs[b] if multi_modal_inputs is not None else None
        grid = mm.get("image_grid_thw") if isinstance(mm, dict) else None
        vgrid = mm.get("video_grid_thw") if isinstance(mm, dict) else None
        p3, _ = get_rope_index(input_ids[b][m], grid, image_token_id, merge_size, video_grid_thw=vgrid,
                               video_token_id=video_token_id)
        out[b, 1:, m] = p3
    return out
