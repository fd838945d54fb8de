"""Semantic token streams (video latent frames, action chunks, text + proprio) that select the per-row
gain of a quantized linear.  Mirrors the reference's ``streams.py:10-120``."""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class FastWAMStreamConfig:
    video_latent_frames: int = 3
    action_chunks: int = 2
    proprio_tokens: int = 1
    split_context: bool = True

    def validate(self) -> None:
        if self.video_latent_frames <= 0 or self.action_chunks <= 0:
            raise ValueError("video_latent_frames and action_chunks must be positive.")
        if self.proprio_tokens < 0:
            raise ValueError("proprio_tokens must be non-negative.")


@dataclass(frozen=True)
class ResolvedStreamLayout:
    names: tuple[str, ...]
    token_counts: tuple[int, ...]

    @property
    def num_streams(self) -> int:
        return len(self.names)

    def validate(self, sequence_length: int) -> None:
        if not self.names or len(self.names) != len(self.token_counts):
            raise ValueError("A stream layout needs one non-empty name per token count.")
        if min(self.token_counts) <= 0:
            raise ValueError("Every stream must contain at least one token.")
        if sum(self.token_counts) != int(sequence_length):
            raise ValueError("Stream token counts do not cover the input sequence.")

    def slices(self) -> tuple[slice, ...]:
        edges = [0]
        for count in self.token_counts:
            edges.append(edges[-1] + count)
        return tuple(slice(a, b) for a, b in zip(edges[:-1], edges[1:]))


def _equal(prefix: str, length: int, parts: int) -> ResolvedStreamLayout:
    if length % parts:
        raise ValueError(f"Sequence length {length} is not divisible by {parts} {prefix} streams.")
    return ResolvedStreamLayout(tuple(f"{prefix}_{i}" for i in range(parts)), (length // parts,) * parts)


def resolve_stream_layout(site, sequence_length: int, config: FastWAMStreamConfig) -> ResolvedStreamLayout:
    """Layout of one site's token axis (``streams.py:68-94``): context sites split into text + proprio,
    video sites into latent frames, action sites into action chunks."""
    config.validate()
    length = int(sequence_length)
    if length <= 0:
        raise ValueError("sequence_length must be positive.")
    if site.stream_kind == "context":
        if config.split_context and config.proprio_tokens > 0:
            text = length - config.proprio_tokens
            if text <= 0:
                raise ValueError("Context must contain text tokens before appended proprio tokens.")
            layout = ResolvedStreamLayout(("text", "proprio"), (text, config.proprio_tokens))
        else:
            layout = ResolvedStreamLayout(("context",), (length,))
    elif site.expert == "video":
        layout = _equal("latent_frame", length, config.video_latent_frames)
    else:
        layout = _equal("action_chunk", length, config.action_chunks)
    layout.validate(length)
    return layout


def rows_for_stream(x: torch.Tensor, stream_slice: slice) -> torch.Tensor:
    if x.ndim < 2:
        raise ValueError("Linear input must have a token and hidden dimension.")
    picked = x[..., stream_slice, :]
    return picked.reshape(-1, picked.shape[-1])


def expand_stream_gains(x: torch.Tensor, gains: torch.Tensor, layout: ResolvedStreamLayout) -> torch.Tensor:
    """One gain per stream -> one gain per token row, shaped to broadcast against ``x``
    (``streams.py:104-120``)."""
    if x.ndim < 2 or x.shape[-2] != sum(layout.token_counts):
        raise ValueError("Runtime tensor does not match its stream layout.")
    gains = torch.as_tensor(gains, device=x.device, dtype=x.dtype)
    if gains.shape != (layout.num_streams,):
        raise ValueError(f"Expected {layout.num_streams} gains, got {tuple(gains.shape)}.")
    per_row = torch.repeat_interleave(gains, torch.tensor(layout.token_counts, device=x.device))
    view = [1] * x.ndim
    view[-2] = x.shape[-2]
    return per_row.reshape(view)
