"""Choosing and decoding video frames (CPU).

``sample_timestamps`` decides *when* to sample: about ``fps`` frames per second, at least ``min_frames`` and
at most ``max_frames``, spread evenly over the clip with both end points included.  ``decode_video_frames``
reads those frames with PyAV in one forward pass over the stream; PyAV is optional and imported on use.
Parity: kempnerforge/data/video_io.py:36-127 (registered sampling policy ``"uniform"``, same clamping and
end-point rules; frames come back as PIL images so the still-image preprocessing is reused).
"""

from __future__ import annotations

from typing import Any

from kempnerforge_b200.config.registry import registry


def sample_timestamps(duration_s: float, fps: float, min_frames: int, max_frames: int) -> list[float]:
    """Strictly increasing sample times in seconds, between 1 and ``max_frames`` of them."""
    if fps <= 0:
        raise ValueError(f"fps must be positive (got {fps})")
    if min_frames < 1 or max_frames < 1:
        raise ValueError(f"min_frames and max_frames must be >= 1 (got {min_frames}, {max_frames})")
    if min_frames > max_frames:
        raise ValueError(f"min_frames ({min_frames}) must be <= max_frames ({max_frames})")
    if duration_s <= 0.0:
        return [0.0]
    count = min(max(round(duration_s * fps), min_frames), max_frames)
    if count <= 1:
        return [0.0]
    return [duration_s * i / (count - 1) for i in range(count)]


registry.register("sampling_policy", "uniform", sample_timestamps)


def clip_duration_seconds(stream: Any, container: Any) -> float:
    """Clip length from whichever piece of metadata the container carries (0.0 when unknown)."""
    if getattr(stream, "duration", None) is not None and getattr(stream, "time_base", None) is not None:
        return float(stream.duration * stream.time_base)
    if getattr(container, "duration", None) is not None:
        return float(container.duration) / 1e6  # container durations are in microseconds
    if getattr(stream, "frames", 0) and getattr(stream, "average_rate", None):
        return float(stream.frames) / float(stream.average_rate)
    return 0.0


def pick_frames(frames, targets: list[float], eps: float = 1e-3) -> list[Any]:
    """From an iterator of (time_s, frame) in presentation order take, for every target time, the first frame
    at or after it; targets beyond the end get the last frame.  Stops reading once all targets are served."""
    chosen: list[Any] = []
    last = None
    it = iter(frames)
    for t, frame in it:
        while len(chosen) < len(targets) and t + eps >= targets[len(chosen)]:
            chosen.append(frame)
        last = frame
        if len(chosen) == len(targets):
            break
    if last is not None:
        chosen.extend(last for _ in range(len(targets) - len(chosen)))
    return chosen


def decode_video_frames(path: str, *, fps: float, min_frames: int, max_frames: int,
                        sampling_policy: str = "uniform") -> list[Any]:
    """RGB ``PIL.Image`` frames of the clip at ``path``; empty when it has no video stream."""
    try:
        import av
    except ImportError as e:  # pragma: no cover
        raise ImportError("decoding video needs the optional PyAV package (`pip install av`)") from e
    policy = registry.get("sampling_policy", sampling_policy)
    with av.open(path) as container:
        if not container.streams.video:
            return []
        stream = container.streams.video[0]
        stream.thread_type = "AUTO"
        targets = policy(clip_duration_seconds(stream, container), fps, min_frames, max_frames)
        timed = ((float(f.time) if f.time is not None else 0.0, f) for f in container.decode(stream))
        return [f.to_image() for f in pick_frames(timed, targets)]
