"""Multimodal input plugin: turns ``<image>`` / ``<video>`` placeholders of chat messages into the right number of
vision tokens and produces the pixel tensors the vision tower consumes.

Plugins: ``base`` (text only: rejects media), ``qwen2_vl`` (Qwen2-VL / Qwen2.5-VL; the hybrid VL models of this
project) and ``qwen3_vl`` (adds per-frame timestamps for videos).  The image pipeline is self-contained (PIL + torch):
resize to a pixel budget on a ``patch * merge`` grid, normalise, cut into ``[grid_t * grid_h * grid_w,
C * temporal_patch * patch * patch]`` rows in the merge-block order the Qwen2-VL vision tower expects.

Reference: ``data/mm_plugin.py`` (``Qwen2VLPlugin`` at lines 1469-1609, ``Qwen3VLPlugin`` 1611-1732, registry at
2222-2241); the reference delegates the pixel work to the HF image / video processors.
"""
from __future__ import annotations

import math
from copy import deepcopy
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Union

import torch

IMAGE_PLACEHOLDER = "<image>"
VIDEO_PLACEHOLDER = "<video>"
AUDIO_PLACEHOLDER = "<audio>"

ImageInput = Union[str, bytes, dict, "PIL.Image.Image", torch.Tensor]     # noqa: F821


@dataclass
class VisionProcessorConfig:
    """The few numbers of an HF Qwen2-VL image processor that matter here."""
    patch_size: int = 14
    temporal_patch_size: int = 2
    merge_size: int = 2
    image_mean: Sequence[float] = (0.48145466, 0.4578275, 0.40821073)
    image_std: Sequence[float] = (0.26862954, 0.26130258, 0.27577711)
    image_max_pixels: int = 768 * 768
    image_min_pixels: int = 32 * 32
    video_max_pixels: int = 256 * 256
    video_min_pixels: int = 16 * 16
    video_fps: float = 2.0
    video_maxlen: int = 128


def smart_resize(height: int, width: int, factor: int, min_pixels: int, max_pixels: int):
    """Height / width rounded to multiples of ``factor`` with the area inside ``[min_pixels, max_pixels]`` and the
    aspect ratio kept as far as the grid allows."""
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def _open_image(image: ImageInput):
    from PIL import Image
    if isinstance(image, Image.Image):
        return image
    if isinstance(image, torch.Tensor):       # [C, H, W] or [H, W, C], 0..1 floats or uint8
        t = image
        if t.dim() == 3 and t.shape[0] in (1, 3) and t.shape[-1] not in (1, 3):
            t = t.permute(1, 2, 0)
        if t.is_floating_point():
            t = (t.clamp(0, 1) * 255).round()
        return Image.fromarray(t.to(torch.uint8).cpu().numpy().squeeze())
    if isinstance(image, bytes):
        import io
        return Image.open(io.BytesIO(image))
    if isinstance(image, dict):
        if image.get("bytes") is not None:
            import io
            return Image.open(io.BytesIO(image["bytes"]))
        return Image.open(image["path"])
    return Image.open(image)


class BasePlugin:
    """Text-only plugin: validates that no media is passed; the interface every plugin implements."""

    def __init__(self, image_token: Optional[str] = None, video_token: Optional[str] = None,
                 audio_token: Optional[str] = None, expand_mm_tokens: bool = True):
        self.image_token, self.video_token, self.audio_token = image_token, video_token, audio_token
        self.expand_mm_tokens = expand_mm_tokens

    def _validate(self, messages, images, videos, audios) -> None:
        for kind, items, tok in (("image", images, self.image_token), ("video", videos, self.video_token),
                                 ("audio", audios, self.audio_token)):
            if items and tok is None:
                raise ValueError(f"this model does not take {kind} inputs")
        text = "".join(m["content"] for m in messages)
        for ph, items, kind in ((IMAGE_PLACEHOLDER, images, "image"), (VIDEO_PLACEHOLDER, videos, "video"),
                                (AUDIO_PLACEHOLDER, audios, "audio")):
            if text.count(ph) != len(items or []):
                raise ValueError(f"{len(items or [])} {kind}(s) given but the messages hold {text.count(ph)} {ph} placeholders")

    def process_messages(self, messages: List[Dict[str, str]], images=(), videos=(), audios=(), processor=None):
        self._validate(messages, images, videos, audios)
        return messages

    def process_token_ids(self, input_ids: List[int], labels: Optional[List[int]], images=(), videos=(), audios=(),
                          tokenizer=None, processor=None):
        return input_ids, labels

    def get_mm_inputs(self, images=(), videos=(), audios=(), processor=None, **_) -> Dict[str, torch.Tensor]:
        if images or videos or audios:
            raise ValueError("this model does not take multimodal inputs")
        return {}


class Qwen2VLPlugin(BasePlugin):
    vision_bos_token = "<|vision_start|>"
    vision_eos_token = "<|vision_end|>"

    # -- images ------------------------------------------------------------------------------------
    def _preprocess_image(self, image, max_pixels: int, min_pixels: int):
        img = _open_image(image)
        if img.mode != "RGB":
            img = img.convert("RGB")
        if min(img.width, img.height) < 28:                     # the tower needs at least one merged patch per side
            img = img.resize((max(img.width, 28), max(img.height, 28)))
        if img.width / img.height > 200:                        # extreme panoramas are squeezed to 180:1
            img = img.resize((img.height * 180, img.height))
        if img.height / img.width > 200:
            img = img.resize((img.width, img.width * 180))
        return img

    def _patchify(self, frames: List, cfg: VisionProcessorConfig, max_pixels: int, min_pixels: int):
        """``frames``: PIL images of one image (1 frame) or one video.  Returns ``(rows, (t, h, w))``."""
        import numpy as np
        from PIL import Image
        ps, tps, ms = cfg.patch_size, cfg.temporal_patch_size, cfg.merge_size
        H, W = smart_resize(frames[0].height, frames[0].width, ps * ms, min_pixels, max_pixels)
        mean = torch.tensor(cfg.image_mean).view(1, 3, 1, 1)
        std = torch.tensor(cfg.image_std).view(1, 3, 1, 1)
        arr = np.stack([np.asarray(f.resize((W, H), Image.BICUBIC), dtype=np.float32) / 255.0 for f in frames])
        x = (torch.from_numpy(arr).permute(0, 3, 1, 2) - mean) / std           # [T, 3, H, W]
        if x.shape[0] % tps:
            x = torch.cat([x, x[-1:].expand(tps - x.shape[0] % tps, -1, -1, -1)])
        gt, gh, gw = x.shape[0] // tps, H // ps, W // ps
        x = x.reshape(gt, tps, 3, gh // ms, ms, ps, gw // ms, ms, ps)
        x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)                                # t, h', w', mh, mw, C, tp, ph, pw
        return x.reshape(gt * gh * gw, 3 * tps * ps * ps).contiguous(), (gt, gh, gw)

    # -- videos ------------------------------------------------------------------------------------
    def _sample_indices(self, total_frames: int, native_fps: float, cfg: VisionProcessorConfig) -> List[int]:
        n = min(cfg.video_maxlen, max(1, int(total_frames / max(native_fps, 1e-6) * cfg.video_fps)), total_frames)
        return [round(i * (total_frames - 1) / max(n - 1, 1)) for i in range(n)]

    def _video_frames(self, video, cfg: VisionProcessorConfig):
        """A video is a list of frames (images / paths) or a path to a container (needs PyAV)."""
        if isinstance(video, (list, tuple)):
            frames = [self._preprocess_image(f, cfg.video_max_pixels, cfg.video_min_pixels) for f in video]
            fps = cfg.video_fps
        else:
            try:
                import av
            except ImportError as e:       # pragma: no cover - optional dependency
                raise RuntimeError("decoding a video file needs the `av` package; pass a list of frames instead") from e
            container = av.open(video, "r")
            stream = next(s for s in container.streams if s.type == "video")
            idx = set(self._sample_indices(stream.frames, float(stream.average_rate), cfg))
            frames = [self._preprocess_image(f.to_image(), cfg.video_max_pixels, cfg.video_min_pixels)
                      for i, f in enumerate(container.decode(stream)) if i in idx]
            dur = float(stream.duration * stream.time_base) if stream.duration else len(frames) / cfg.video_fps
            fps = len(frames) / max(dur, 1e-6)
        if len(frames) % 2:
            frames.append(frames[-1])
        return frames, fps

    # -- tensors -----------------------------------------------------------------------------------
    def get_mm_inputs(self, images=(), videos=(), audios=(), processor: Optional[VisionProcessorConfig] = None, **_):
        cfg = processor or VisionProcessorConfig()
        if audios:
            raise ValueError("this model does not take audio inputs")
        out: Dict[str, torch.Tensor] = {}
        if images:
            rows, grids = [], []
            for im in images:
                r, g = self._patchify([self._preprocess_image(im, cfg.image_max_pixels, cfg.image_min_pixels)], cfg,
                                      cfg.image_max_pixels, cfg.image_min_pixels)
                rows.append(r)
                grids.append(g)
            out["pixel_values"], out["image_grid_thw"] = torch.cat(rows), torch.tensor(grids, dtype=torch.long)
        if videos:
            rows, grids, secs = [], [], []
            for vid in videos:
                frames, fps = self._video_frames(vid, cfg)
                r, g = self._patchify(frames, cfg, cfg.video_max_pixels, cfg.video_min_pixels)
                rows.append(r)
                grids.append(g)
                secs.append(cfg.temporal_patch_size / fps)
            out["pixel_values_videos"], out["video_grid_thw"] = torch.cat(rows), torch.tensor(grids, dtype=torch.long)
            out["second_per_grid_ts"] = secs
        return out

    # -- text --------------------------------------------------------------------------------------
    def _video_block(self, n_tokens: int, grid, seconds_per_grid: float) -> str:
        return f"{self.vision_bos_token}{self.video_token * n_tokens}{self.vision_eos_token}"

    def process_messages(self, messages, images=(), videos=(), audios=(), processor=None):
        self._validate(messages, images, videos, audios)
        cfg = processor or VisionProcessorConfig()
        merge = cfg.merge_size ** 2
        mm = self.get_mm_inputs(images, videos, audios, cfg) if self.expand_mm_tokens and (images or videos) else {}
        ig, vg = mm.get("image_grid_thw"), mm.get("video_grid_thw")
        secs = mm.get("second_per_grid_ts", [])
        messages = deepcopy(messages)
        ni = nv = 0
        for m in messages:
            c = m["content"]
            while IMAGE_PLACEHOLDER in c:
                n = int(ig[ni].prod()) // merge if ig is not None else 1
                c = c.replace(IMAGE_PLACEHOLDER, f"{self.vision_bos_token}{self.image_token * n}{self.vision_eos_token}", 1)
                ni += 1
            while VIDEO_PLACEHOLDER in c:
                n = int(vg[nv].prod()) // merge if vg is not None else 1
                c = c.replace(VIDEO_PLACEHOLDER, self._video_block(n, None if vg is None else vg[nv],
                                                                   secs[nv] if secs else 0.0), 1)
                nv += 1
            m["content"] = c
        return messages


class Qwen3VLPlugin(Qwen2VLPlugin):
    """Videos are written frame group by frame group, each preceded by its timestamp (``<1.5 seconds>``)."""

    def _video_block(self, n_tokens: int, grid, seconds_per_grid: float) -> str:
        if grid is None:
            return super()._video_block(n_tokens, grid, seconds_per_grid)
        gt = int(grid[0])
        per = n_tokens // gt
        parts = []
        for t in range(gt):
            stamp = (t + 0.5) * seconds_per_grid
            parts.append(f"<{stamp:.1f} seconds>{self.vision_bos_token}{self.video_token * per}{self.vision_eos_token}")
        return "".join(parts)


PLUGINS = {"base": BasePlugin, "qwen2_vl": Qwen2VLPlugin, "qwen3_vl": Qwen3VLPlugin}


def register_mm_plugin(name: str, plugin_class: type) -> None:
    if name in PLUGINS:
        raise ValueError(f"multimodal plugin {name} already exists")
    PLUGINS[name] = plugin_class


def get_mm_plugin(name: str, image_token: Optional[str] = None, video_token: Optional[str] = None,
                  audio_token: Optional[str] = None, **kw) -> BasePlugin:
    if name not in PLUGINS:
        from . import mm_plugin_audio, mm_plugin_zoo  # noqa: F401  (register the other families' plugins)
    if name not in PLUGINS:
        raise ValueError(f"multimodal plugin `{name}` not found")
    return PLUGINS[name](image_token, video_token, audio_token, **kw)
