"""Multimodal plugins of further model families: how many vision tokens an ``<image>`` / ``<video>`` placeholder
becomes, which wrapper tokens surround them, and the pixel tensor the family's vision tower takes.

Each plugin restates the token layout its family prescribes; the pixel work is the same self-contained pipeline as in
``mm_plugin.py`` (PIL + torch: resize, normalise, optionally tile).  Registered names: ``llava``, ``llava_next``,
``video_llava``, ``paligemma``, ``pixtral``, ``intern_vl``, ``gemma3``, ``glm4v``, ``mllama``.
Reference: the plugin classes of ``data/mm_plugin.py`` (``LlavaPlugin`` 862-896, ``LlavaNextPlugin`` 898-936,
``PaliGemmaPlugin`` 1280-1343, ``PixtralPlugin`` 1345-1412, ``InternVLPlugin`` 613-761, ``Gemma3Plugin`` 520-577,
``GLM4VPlugin`` 1734-1863, ``MllamaPlugin`` 1225-1278, ``VideoLlavaPlugin`` 2043-2094)."""
from __future__ import annotations

import math
from copy import deepcopy
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .mm_plugin import (IMAGE_PLACEHOLDER, VIDEO_PLACEHOLDER, BasePlugin, Qwen2VLPlugin, _open_image,
                        register_mm_plugin)

IGNORE_INDEX = -100


@dataclass
class TowerConfig:
    """Numbers of a fixed-resolution vision tower (CLIP / SigLIP style)."""
    image_size: int = 336
    patch_size: int = 14
    image_mean: Sequence[float] = (0.48145466, 0.4578275, 0.40821073)
    image_std: Sequence[float] = (0.26862954, 0.26130258, 0.27577711)
    has_cls_token: bool = False          # towers with a class token and "full" feature selection emit one more token
    video_frames: int = 8
    max_tiles: int = 12                  # dynamic tiling (InternVL)
    grid_pinpoints: Sequence[Tuple[int, int]] = ((336, 672), (672, 336), (672, 672), (1008, 336), (336, 1008))

    @property
    def tokens_per_side(self) -> int:
        return self.image_size // self.patch_size

    @property
    def image_seqlen(self) -> int:
        return self.tokens_per_side ** 2 + (1 if self.has_cls_token else 0)


def _to_tensor(img, size: Tuple[int, int], cfg: TowerConfig) -> torch.Tensor:
    """PIL image -> normalised ``[3, H, W]`` float tensor at ``size = (H, W)``."""
    import numpy as np
    from PIL import Image
    if img.mode != "RGB":
        img = img.convert("RGB")
    arr = np.asarray(img.resize((size[1], size[0]), Image.BICUBIC), dtype=np.float32) / 255.0
    x = torch.from_numpy(arr).permute(2, 0, 1)
    mean = torch.tensor(cfg.image_mean).view(3, 1, 1)
    std = torch.tensor(cfg.image_std).view(3, 1, 1)
    return (x - mean) / std


def _replace_each(content: str, placeholder: str, blocks: List[str], cursor: int) -> Tuple[str, int]:
    while placeholder in content:
        content = content.replace(placeholder, blocks[cursor], 1)
        cursor += 1
    return content, cursor


class LlavaPlugin(BasePlugin):
    """Every image is resized to the tower's square input and becomes ``image_seqlen`` copies of the image token."""

    def _image_block(self, img, cfg: TowerConfig) -> str:
        return self.image_token * cfg.image_seqlen

    def process_messages(self, messages, images=(), videos=(), audios=(), processor=None):
        self._validate(messages, images, videos, audios)
        cfg = processor or TowerConfig()
        blocks = [self._image_block(_open_image(i), cfg) if self.expand_mm_tokens else self.image_token for i in images]
        messages = deepcopy(messages)
        cur = 0
        for m in messages:
            m["content"], cur = _replace_each(m["content"], IMAGE_PLACEHOLDER, blocks, cur)
        return messages

    def get_mm_inputs(self, images=(), videos=(), audios=(), processor=None, **_) -> Dict[str, torch.Tensor]:
        if not images:
            return {}
        cfg = processor or TowerConfig()
        px = [_to_tensor(_open_image(i), (cfg.image_size, cfg.image_size), cfg) for i in images]
        return {"pixel_values": torch.stack(px)}


def select_best_resolution(size: Tuple[int, int], candidates: Sequence[Tuple[int, int]]) -> Tuple[int, int]:
    """The candidate ``(H, W)`` that keeps most of the image's pixels after an aspect-preserving fit, ties broken by
    the least wasted area."""
    h, w = size
    best, best_eff, best_waste = None, -1, None
    for ch, cw in candidates:
        scale = min(cw / w, ch / h)
        eff = min(int(w * scale) * int(h * scale), w * h)
        waste = ch * cw - eff
        if eff > best_eff or (eff == best_eff and waste < best_waste):
            best, best_eff, best_waste = (ch, cw), eff, waste
    return best


class LlavaNextPlugin(LlavaPlugin):
    """"Any resolution": the image is fitted into the best of a few canvas sizes and cut into tower-sized tiles; the
    token count is the base image's features plus the un-padded tile features with one newline token per row."""

    def _counts(self, height: int, width: int, cfg: TowerConfig) -> int:
        side = cfg.tokens_per_side
        bh, bw = select_best_resolution((height, width), cfg.grid_pinpoints)
        gh, gw = bh // cfg.image_size, bw // cfg.image_size
        cur_h, cur_w = gh * side, gw * side
        # features that cover padding are dropped: the kept region has the image's aspect ratio
        if width / height > cur_w / cur_h:
            new_h = int(round(height * (cur_w / width), 7))
            cur_h -= 2 * ((cur_h - new_h) // 2)
        else:
            new_w = int(round(width * (cur_h / height), 7))
            cur_w -= 2 * ((cur_w - new_w) // 2)
        return side * side + cur_h * cur_w + cur_h          # base + tiles + one newline per feature row

    def _image_block(self, img, cfg: TowerConfig) -> str:
        return self.image_token * self._counts(img.height, img.width, cfg)

    def get_mm_inputs(self, images=(), videos=(), audios=(), processor=None, **_) -> Dict[str, torch.Tensor]:
        if not images:
            return {}
        cfg = processor or TowerConfig()
        out, sizes = [], []
        for i in images:
            img = _open_image(i)
            bh, bw = select_best_resolution((img.height, img.width), cfg.grid_pinpoints)
            canvas = _to_tensor(img, (bh, bw), cfg)
            tiles = [_to_tensor(img, (cfg.image_size, cfg.image_size), cfg)]
            for r in range(bh // cfg.image_size):
                for c in range(bw // cfg.image_size):
                    tiles.append(canvas[:, r * cfg.image_size:(r + 1) * cfg.image_size,
                                        c * cfg.image_size:(c + 1) * cfg.image_size])
            out.append(torch.stack(tiles))
            sizes.append([img.height, img.width])
        n = max(t.shape[0] for t in out)
        padded = torch.zeros(len(out), n, *out[0].shape[1:])
        for j, t in enumerate(out):
            padded[j, :t.shape[0]] = t
        return {"pixel_values": padded, "image_sizes": torch.tensor(sizes)}


class VideoLlavaPlugin(LlavaPlugin):
    """Images as in LLaVA (with the tower's class token kept: one more token); a video is ``video_frames`` uniformly
    sampled frames, each as many video tokens."""

    def process_messages(self, messages, images=(), videos=(), audios=(), processor=None):
        cfg = processor or TowerConfig(image_size=224, has_cls_token=True)
        messages = super().process_messages(messages, images, videos, audios, cfg)
        n = cfg.image_seqlen * cfg.video_frames if self.expand_mm_tokens else 1
        for m in messages:
            m["content"] = m["content"].replace(VIDEO_PLACEHOLDER, self.video_token * n)
        return messages

    def get_mm_inputs(self, images=(), videos=(), audios=(), processor=None, **_) -> Dict[str, torch.Tensor]:
        cfg = processor or TowerConfig(image_size=224, has_cls_token=True)
        out = super().get_mm_inputs(images, (), (), cfg)
        clips = []
        for frames in videos:           # a video is given as a list of frames (decoding is the caller's business)
            idx = torch.linspace(0, len(frames) - 1, cfg.video_frames).round().long().tolist()
            clips.append(torch.stack([_to_tensor(_open_image(frames[j]), (cfg.image_size, cfg.image_size), cfg)
                                      for j in idx]))
        if clips:
            out["pixel_values_videos"] = torch.stack(clips)
        return out


class PaliGemmaPlugin(LlavaPlugin):
    """The image tokens do not stand where the placeholder was: the placeholders are removed and ``image_seqlen`` image
    tokens per image are put in front of the whole prompt (never trained on); ``token_type_ids`` mark the prefix."""

    def process_messages(self, messages, images=(), videos=(), audios=(), processor=None):
        self._validate(messages, images, videos, audios)
        messages = deepcopy(messages)
        for m in messages:
            m["content"] = m["content"].replace(IMAGE_PLACEHOLDER, "")
        return messages

    def process_token_ids(self, input_ids, labels, images=(), videos=(), audios=(), tokenizer=None, processor=None):
        cfg = processor or TowerConfig(image_size=224)
        n = len(images) * cfg.image_seqlen if self.expand_mm_tokens else len(images)
        tok = tokenizer.convert_tokens_to_ids(self.image_token)
        input_ids = [tok] * n + list(input_ids)
        if labels is not None:
            labels = [IGNORE_INDEX] * n + list(labels)
        return input_ids, labels

    def get_mm_inputs(self, images=(), videos=(), audios=(), processor=None, seqlens: Sequence[int] = (), **_):
        cfg = processor or TowerConfig(image_size=224)
        out = super().get_mm_inputs(images, (), (), cfg)
        if seqlens:         # 0 for the image prefix and the prompt, set by the collator per sample
            n = len(images) * cfg.image_seqlen
            out["token_type_ids"] = torch.tensor([[0] * n + [1] * (s - n) for s in seqlens])
        return out


class PixtralPlugin(LlavaPlugin):
    """Images keep their aspect ratio (longest side at most ``image_size``); every row of patches is written as image
    tokens followed by a row-break token, the last row ends with the image-end token."""
    break_token, end_token = "[IMG_BREAK]", "[IMG_END]"

    def _grid(self, img, cfg: TowerConfig) -> Tuple[int, int]:
        ratio = max(img.height / cfg.image_size, img.width / cfg.image_size)
        h, w = img.height, img.width
        if ratio > 1:                  # rounded down, so that the longest side never exceeds the limit
            h, w = int(math.floor(h / ratio)), int(math.floor(w / ratio))
        return max(1, (h - 1) // cfg.patch_size + 1), max(1, (w - 1) // cfg.patch_size + 1)

    def _image_block(self, img, cfg: TowerConfig) -> str:
        gh, gw = self._grid(img, cfg)
        rows = [self.image_token * gw + self.break_token] * gh
        rows[-1] = self.image_token * gw + self.end_token
        return "".join(rows)

    def process_messages(self, messages, images=(), videos=(), audios=(), processor=None):
        return super().process_messages(messages, images, videos, audios, processor or TowerConfig(image_size=1024, patch_size=16))

    def get_mm_inputs(self, images=(), videos=(), audios=(), processor=None, **_):
        if not images:
            return {}
        cfg = processor or TowerConfig(image_size=1024, patch_size=16)
        px, sizes = [], []
        for i in images:
            img = _open_image(i)
            gh, gw = self._grid(img, cfg)
            px.append(_to_tensor(img, (gh * cfg.patch_size, gw * cfg.patch_size), cfg))
            sizes.append([gh * cfg.patch_size, gw * cfg.patch_size])
        return {"pixel_values": px, "image_sizes": torch.tensor(sizes)}        # ragged: a list of [3, H, W]


class InternVLPlugin(LlavaPlugin):
    """Dynamic tiling: the image is cut into the ``a x b`` grid of tower-sized tiles (``a b <= max_tiles``) whose aspect
    ratio is closest to the image's, plus a thumbnail when there is more than one tile; each tile becomes
    ``image_seqlen`` context tokens (a quarter of the patch count: pixel-shuffle) between ``<img>`` and ``</img>``."""
    start_token, end_token = "<img>", "</img>"

    @staticmethod
    def tile_grid(height: int, width: int, cfg: TowerConfig) -> Tuple[int, int]:
        target = width / height
        grids = sorted({(a, b) for n in range(1, cfg.max_tiles + 1) for a in range(1, n + 1) for b in range(1, n + 1)
                        if a * b <= cfg.max_tiles}, key=lambda g: g[0] * g[1])
        best, best_diff = (1, 1), float("inf")
        for a, b in grids:                       # a columns, b rows
            diff = abs(target - a / b)
            if diff < best_diff or (diff == best_diff and height * width > 0.5 * cfg.image_size ** 2 * a * b):
                best, best_diff = (a, b), diff
        return best

    def _tiles(self, img, cfg: TowerConfig) -> int:
        a, b = self.tile_grid(img.height, img.width, cfg)
        return a * b + (1 if a * b > 1 else 0)

    def _image_block(self, img, cfg: TowerConfig) -> str:
        per_tile = cfg.tokens_per_side ** 2 // 4
        return self.start_token + self.image_token * (per_tile * self._tiles(img, cfg)) + self.end_token

    def process_messages(self, messages, images=(), videos=(), audios=(), processor=None):
        return super().process_messages(messages, images, videos, audios, processor or TowerConfig(image_size=448))

    def get_mm_inputs(self, images=(), videos=(), audios=(), processor=None, **_):
        if not images:
            return {}
        cfg = processor or TowerConfig(image_size=448)
        tiles, counts = [], []
        for i in images:
            img = _open_image(i)
            a, b = self.tile_grid(img.height, img.width, cfg)
            canvas = _to_tensor(img, (b * cfg.image_size, a * cfg.image_size), cfg)
            mine = [canvas[:, r * cfg.image_size:(r + 1) * cfg.image_size, c * cfg.image_size:(c + 1) * cfg.image_size]
                    for r in range(b) for c in range(a)]
            if a * b > 1:
                mine.append(_to_tensor(img, (cfg.image_size, cfg.image_size), cfg))
            tiles += mine
            counts.append(len(mine))
        return {"pixel_values": torch.stack(tiles), "image_num_patches": torch.tensor(counts)}


class Gemma3Plugin(LlavaPlugin):
    """One 896 x 896 view per image, pooled to 256 soft tokens, written between the begin / end markers on lines of
    their own."""
    boi_token, eoi_token = "<start_of_image>", "<end_of_image>"

    def _image_block(self, img, cfg: TowerConfig) -> str:
        return f"\n\n{self.boi_token}{self.image_token * 256}{self.eoi_token}\n\n"

    def process_messages(self, messages, images=(), videos=(), audios=(), processor=None):
        return super().process_messages(messages, images, videos, audios, processor or TowerConfig(image_size=896))

    def get_mm_inputs(self, images=(), videos=(), audios=(), processor=None, **_):
        return super().get_mm_inputs(images, videos, audios, processor or TowerConfig(
            image_size=896, image_mean=(0.5, 0.5, 0.5), image_std=(0.5, 0.5, 0.5)))


class GLM4VPlugin(Qwen2VLPlugin):
    """The Qwen2-VL pipeline (dynamic resolution on a patch-merge grid) with this family's begin / end markers."""
    vision_bos_token = "<|begin_of_image|>"
    vision_eos_token = "<|end_of_image|>"

    def _video_block(self, n_tokens: int, grid, seconds_per_grid: float) -> str:
        if grid is None:
            return f"<|begin_of_video|>{self.video_token * n_tokens}<|end_of_video|>"
        gt = int(grid[0])
        per = n_tokens // gt
        frames = "".join(f"{self.vision_bos_token}{self.image_token * per}{self.vision_eos_token}{int(t * seconds_per_grid)}"
                         for t in range(gt))
        return f"<|begin_of_video|>{frames}<|end_of_video|>"


class MllamaPlugin(LlavaPlugin):
    """One image token per image (the pixels enter through cross-attention); ``cross_attention_mask`` tells every text
    token which images precede it."""

    def _image_block(self, img, cfg: TowerConfig) -> str:
        return self.image_token

    def get_mm_inputs(self, images=(), videos=(), audios=(), processor=None, batch_ids: Sequence[Sequence[int]] = (),
                      image_token_id: Optional[int] = None, **_):
        cfg = processor or TowerConfig(image_size=560)
        out = super().get_mm_inputs(images, (), (), cfg)
        if batch_ids and image_token_id is not None:
            n_img = max(1, max(sum(t == image_token_id for t in ids) for ids in batch_ids))
            L = max(len(ids) for ids in batch_ids)
            mask = torch.zeros(len(batch_ids), L, n_img, dtype=torch.long)
            for b, ids in enumerate(batch_ids):
                seen = -1
                for t, tok in enumerate(ids):
                    if tok == image_token_id:
                        seen += 1
                    if seen >= 0:
                        mask[b, t, :seen + 1] = 1       # a token sees every image that came before it
            out["cross_attention_mask"] = mask
        return out


for _name, _cls in (("llava", LlavaPlugin), ("llava_next", LlavaNextPlugin), ("video_llava", VideoLlavaPlugin),
                    ("paligemma", PaliGemmaPlugin), ("pixtral", PixtralPlugin), ("intern_vl", InternVLPlugin),
                    ("gemma3", Gemma3Plugin), ("glm4v", GLM4VPlugin), ("mllama", MllamaPlugin)):
    register_mm_plugin(_name, _cls)
