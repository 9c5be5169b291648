"""Audio inputs for speech-language models: a waveform becomes a log-mel spectrogram of fixed length (the input of a
Whisper-style encoder) with a mask of the frames that hold sound, and each ``<audio>`` placeholder in the text becomes
as many audio tokens as the encoder emits for that clip, wrapped in begin / end tokens.

The whole front end is torch: reading PCM ``.wav`` files with the standard library, linear resampling, a Hann-window
STFT, a Slaney-scale triangular mel filter bank, ``log10`` with an 80 dB floor below the clip's maximum, scaled to about
[-1, 1].  The encoder halves the frame rate twice (a stride-2 convolution and a stride-2 pooling), hence the token
count ``((frames - 1) // 2 + 1 - 2) // 2 + 1``.

Registered names: ``qwen2_audio`` (audio only) and ``qwen2_omni`` (the Qwen2-VL image / video rules plus audio; audio
tracks inside videos are not interleaved with the frames here).
Reference: ``data/mm_plugin.py`` ``Qwen2AudioPlugin`` (1414-1470: token count from ``feature_attention_mask``) and
``Qwen2OmniPlugin`` (1600-1732), whose feature extraction is delegated to ``transformers``' ``WhisperFeatureExtractor``
and whose file reading is delegated to ``librosa``."""
from __future__ import annotations

import math
import wave
from copy import deepcopy
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from .mm_plugin import AUDIO_PLACEHOLDER, BasePlugin, Qwen2VLPlugin, register_mm_plugin


@dataclass
class AudioFrontendConfig:
    sampling_rate: int = 16000
    n_fft: int = 400
    hop_length: int = 160
    n_mels: int = 128
    chunk_seconds: float = 30.0
    audio_bos_token: str = "<|audio_bos|>"
    audio_eos_token: str = "<|audio_eos|>"

    @property
    def frames(self) -> int:
        return int(self.chunk_seconds * self.sampling_rate) // self.hop_length


def _hz_to_mel(f: torch.Tensor) -> torch.Tensor:
    """Slaney scale: linear below 1 kHz, logarithmic above."""
    lin = f / (200.0 / 3)
    log = 15.0 + torch.log(f.clamp_min(1e-10) / 1000.0) / (math.log(6.4) / 27.0)
    return torch.where(f >= 1000.0, log, lin)


def _mel_to_hz(m: torch.Tensor) -> torch.Tensor:
    lin = m * (200.0 / 3)
    log = 1000.0 * torch.exp((m - 15.0) * (math.log(6.4) / 27.0))
    return torch.where(m >= 15.0, log, lin)


def mel_filterbank(n_mels: int, n_fft: int, sampling_rate: int) -> torch.Tensor:
    """``[n_mels, n_fft // 2 + 1]`` triangular filters with unit area (Slaney normalisation)."""
    freqs = torch.linspace(0, sampling_rate / 2, n_fft // 2 + 1, dtype=torch.float64)
    top = _hz_to_mel(torch.tensor(sampling_rate / 2.0, dtype=torch.float64))
    edges = _mel_to_hz(torch.linspace(0.0, float(top), n_mels + 2, dtype=torch.float64))
    lower, centre, upper = edges[:-2, None], edges[1:-1, None], edges[2:, None]
    up = (freqs[None] - lower) / (centre - lower)
    down = (upper - freqs[None]) / (upper - centre)
    fb = torch.clamp(torch.minimum(up, down), min=0.0)
    return (fb * (2.0 / (upper - lower))).float()


def load_audio(audio, sampling_rate: int) -> torch.Tensor:
    """Mono float waveform at ``sampling_rate``.  ``audio``: a path to a PCM ``.wav`` file, a 1-D / ``[channels, n]``
    tensor or array already at the target rate, a ``(waveform, rate)`` pair, or a dict with ``array`` and
    ``sampling_rate`` (the layout of dataset audio columns)."""
    rate = sampling_rate
    if isinstance(audio, dict):
        audio, rate = audio["array"], int(audio.get("sampling_rate", sampling_rate))
    elif isinstance(audio, (tuple, list)) and len(audio) == 2 and isinstance(audio[1], (int, float)):
        audio, rate = audio[0], int(audio[1])
    if isinstance(audio, str):
        with wave.open(audio, "rb") as f:
            rate, width, ch = f.getframerate(), f.getsampwidth(), f.getnchannels()
            raw = f.readframes(f.getnframes())
        if width not in (1, 2, 4):
            raise ValueError(f"{audio}: {8 * width}-bit PCM is not supported (8, 16 and 32 are)")
        if width == 1:                                                   # unsigned 8-bit
            x = (torch.frombuffer(bytearray(raw), dtype=torch.uint8).float() - 128.0) / 128.0
        else:
            x = torch.frombuffer(bytearray(raw), dtype={2: torch.int16, 4: torch.int32}[width]).float()
            x = x / float(2 ** (8 * width - 1))
        x = x.reshape(-1, ch).t()
    else:
        x = torch.as_tensor(audio).float()
    if x.dim() == 2:
        x = x.mean(0)
    if x.dim() != 1:
        raise ValueError(f"a waveform has one or two dimensions, not {x.dim()}")
    if rate != sampling_rate and x.numel() > 1:
        n = max(1, int(round(x.numel() * sampling_rate / rate)))
        pos = torch.arange(n, dtype=torch.float64) * (rate / sampling_rate)        # output sample i is at input time i * rate / target
        lo = pos.floor().long().clamp_max(x.numel() - 1)
        hi = (lo + 1).clamp_max(x.numel() - 1)
        frac = (pos - lo).float()
        x = x[lo] * (1 - frac) + x[hi] * frac
    return x


def log_mel(waveform: torch.Tensor, cfg: AudioFrontendConfig) -> Tuple[torch.Tensor, torch.Tensor]:
    """``([n_mels, frames], [frames])``: features of one clip cut / zero-padded to the chunk length, and the mask of
    frames that start inside the clip."""
    n_samples = int(cfg.chunk_seconds * cfg.sampling_rate)
    valid = min(waveform.numel(), n_samples)
    x = torch.zeros(n_samples)
    x[:valid] = waveform[:valid]
    spec = torch.stft(x, cfg.n_fft, cfg.hop_length, window=torch.hann_window(cfg.n_fft), center=True,
                      pad_mode="reflect", return_complex=True)
    power = spec[:, :-1].abs() ** 2                                       # the frame past the end is dropped
    mel = mel_filterbank(cfg.n_mels, cfg.n_fft, cfg.sampling_rate) @ power
    logm = torch.log10(mel.clamp_min(1e-10))
    logm = torch.maximum(logm, logm.max() - 8.0)
    feats = (logm + 4.0) / 4.0
    mask = torch.zeros(cfg.frames, dtype=torch.long)
    mask[:max(1, math.ceil(valid / cfg.hop_length)) if valid else 0] = 1
    return feats, mask


def audio_token_count(n_frames: int) -> int:
    """Tokens the encoder emits for ``n_frames`` valid mel frames (stride-2 convolution, then stride-2 pooling)."""
    after_conv = (n_frames - 1) // 2 + 1
    return max(1, (after_conv - 2) // 2 + 1)


class _AudioMixin:
    """Token expansion and feature tensors for ``<audio>`` placeholders."""

    @staticmethod
    def _audio_cfg(processor) -> AudioFrontendConfig:
        if isinstance(processor, AudioFrontendConfig):
            return processor
        return getattr(processor, "audio", None) or AudioFrontendConfig()

    def _audio_inputs(self, audios, cfg: AudioFrontendConfig) -> Dict[str, torch.Tensor]:
        feats, masks = zip(*[log_mel(load_audio(a, cfg.sampling_rate), cfg) for a in audios])
        return {"input_features": torch.stack(feats), "feature_attention_mask": torch.stack(masks)}

    def _expand_audio(self, messages: List[dict], audios, cfg: AudioFrontendConfig) -> List[dict]:
        if not audios:
            return messages
        if self.expand_mm_tokens:
            lengths = self._audio_inputs(audios, cfg)["feature_attention_mask"].sum(-1).tolist()
        cur = 0
        for m in messages:
            c = m["content"]
            while AUDIO_PLACEHOLDER in c:
                n = audio_token_count(int(lengths[cur])) if self.expand_mm_tokens else 1
                c = c.replace(AUDIO_PLACEHOLDER, f"{cfg.audio_bos_token}{self.audio_token * n}{cfg.audio_eos_token}", 1)
                cur += 1
            m["content"] = c
        return messages


class Qwen2AudioPlugin(_AudioMixin, BasePlugin):
    def process_messages(self, messages, images=(), videos=(), audios=(), processor=None):
        self._validate(messages, images, videos, audios)
        return self._expand_audio(deepcopy(messages), audios, self._audio_cfg(processor))

    def get_mm_inputs(self, images=(), videos=(), audios=(), processor=None, **_) -> Dict[str, torch.Tensor]:
        if images or videos:
            raise ValueError("this model takes audio inputs only")
        return self._audio_inputs(audios, self._audio_cfg(processor)) if audios else {}


class Qwen2OmniPlugin(_AudioMixin, Qwen2VLPlugin):
    """Images and videos as in Qwen2-VL, audio clips as in Qwen2-Audio.  ``processor`` may be a vision configuration
    carrying an ``audio`` attribute, an ``AudioFrontendConfig``, or ``None`` (defaults for both)."""

    @staticmethod
    def _vision_cfg(processor):
        return None if isinstance(processor, AudioFrontendConfig) else processor

    def process_messages(self, messages, images=(), videos=(), audios=(), processor=None):
        self._validate(messages, images, videos, audios)
        vis = Qwen2VLPlugin.process_messages(self, _hide_audio(messages), images, videos, (), self._vision_cfg(processor))
        return self._expand_audio(_show_audio(vis), audios, self._audio_cfg(processor))

    def get_mm_inputs(self, images=(), videos=(), audios=(), processor=None, **kw) -> Dict[str, torch.Tensor]:
        out = Qwen2VLPlugin.get_mm_inputs(self, images, videos, (), self._vision_cfg(processor), **kw) \
            if (images or videos) else {}
        if audios:
            out.update(self._audio_inputs(audios, self._audio_cfg(processor)))
        return out


_HIDDEN = "\x00audio\x00"       # keeps the vision pass (which validates placeholder counts) from seeing audio marks


def _hide_audio(messages: List[dict]) -> List[dict]:
    return [dict(m, content=m["content"].replace(AUDIO_PLACEHOLDER, _HIDDEN)) for m in messages]


def _show_audio(messages: List[dict]) -> List[dict]:
    return [dict(m, content=m["content"].replace(_HIDDEN, AUDIO_PLACEHOLDER)) for m in messages]


for _name, _cls in (("qwen2_audio", Qwen2AudioPlugin), ("qwen2_omni", Qwen2OmniPlugin)):
    register_mm_plugin(_name, _cls)
