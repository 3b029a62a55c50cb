"""Audio inputs for Gemma-4 style models (tunix/processors/audio_processor.py:29-194).

Each `<|audio|>` placeholder token in a prompt is replaced by begin-of-audio, one soft-token placeholder per
audio frame the encoder will emit for that clip, and end-of-audio; the waveforms are padded into
`[batch, clips, samples]` with their true lengths alongside (the encoder masks with them).
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Protocol

import numpy as np

AUDIO_PLACEHOLDER = 258881        # <|audio|>
START_OF_AUDIO = 256000           # begin-of-audio
END_OF_AUDIO = 258883             # end-of-audio
AUDIO_SOFT_TOKEN_PLACEHOLDER = -4
MAX_CLIP_SECONDS = 30


class AudioTokenizerLike(Protocol):
    sample_rate: int

    def get_num_soft_tokens(self, num_samples: int) -> int: ...


@dataclasses.dataclass
class PreprocessedAudioInput:
    audios: np.ndarray              # [batch, clips, samples] float32
    sequence_lengths: np.ndarray    # [batch, clips]


def _as_clip_lists(audios) -> list:
    if isinstance(audios, np.ndarray):
        if audios.ndim != 1:
            raise ValueError("a waveform is a 1-D array")
        return [[audios]]
    if not isinstance(audios, list):
        raise ValueError(f"unsupported audio input {type(audios).__name__}")
    out = []
    for clips in audios:
        if isinstance(clips, np.ndarray):
            clips = [clips]
        if not isinstance(clips, list) or any(not isinstance(c, np.ndarray) or c.ndim != 1 for c in clips):
            raise ValueError("each batch entry is a 1-D waveform or a list of them")
        out.append(clips)
    return out


def process_gemma4_inputs(audios, tokens: list, audio_encoder: AudioTokenizerLike, max_audio_length: Optional[int] = None,
                          max_audio_clips: Optional[int] = None):
    limit = audio_encoder.sample_rate * MAX_CLIP_SECONDS
    if max_audio_length is not None and max_audio_length > limit:
        raise ValueError(f"max_audio_length={max_audio_length} exceeds the {limit}-sample clip limit")
    audios = _as_clip_lists(audios)
    if len(audios) != len(tokens):
        raise ValueError(f"{len(tokens)} token sequences for {len(audios)} audio entries")
    n_clips = [len(c) for c in audios]
    most_clips = max(n_clips) if n_clips else 0
    if max_audio_clips is None:
        max_audio_clips = most_clips
    elif most_clips > max_audio_clips:
        raise ValueError(f"an entry has {most_clips} clips, more than max_audio_clips={max_audio_clips}")
    longest = max((len(c) for clips in audios for c in clips), default=0)
    if max_audio_length is None:
        max_audio_length = longest
        if longest > limit:
            raise ValueError(f"a clip has {longest} samples; the limit is {limit}")
    elif longest > max_audio_length:
        raise ValueError(f"a clip has {longest} samples, more than max_audio_length={max_audio_length}")
    expanded = []
    for b, seq in enumerate(tokens):
        seq = np.asarray(seq).tolist()
        if seq.count(AUDIO_PLACEHOLDER) != n_clips[b]:
            raise ValueError(f"entry {b}: {seq.count(AUDIO_PLACEHOLDER)} audio placeholders for {n_clips[b]} clips")
        out, clip = [], 0
        for t in seq:
            if t == AUDIO_PLACEHOLDER:
                n_soft = audio_encoder.get_num_soft_tokens(len(audios[b][clip]))
                out += [START_OF_AUDIO] + [AUDIO_SOFT_TOKEN_PLACEHOLDER] * n_soft + [END_OF_AUDIO]
                clip += 1
            else:
                out.append(t)
        expanded.append(np.asarray(out))
    processed = None
    if max_audio_clips > 0 and max_audio_length > 0:
        wave = np.zeros((len(audios), max_audio_clips, max_audio_length), np.float32)
        lens = np.zeros((len(audios), max_audio_clips), np.int64)
        for b, clips in enumerate(audios):
            for i, c in enumerate(clips):
                wave[b, i, :len(c)] = c
                lens[b, i] = len(c)
        processed = PreprocessedAudioInput(wave, lens)
    return processed, expanded
