"""Frame access to episode videos by index or by time stamp, behind one interface.

``decode_frames(path, indices=... | timestamps=..., backend=...)`` returns ``[N, H, W, 3]`` uint8 RGB. Backends:

* ``opencv``     — ``cv2.VideoCapture``; sorted requests are served in one forward pass (a seek only when the next frame
  is not the one wanted), which is what makes clips of consecutive frames cheap;
* ``pyav``, ``decord``, ``torchcodec`` — used when the package is installed; asking for one that is not raises an
  ``ImportError`` that names it (none of the three is a dependency of this package).

Time stamps map to the nearest frame of the stream's frame rate; requests past the end return the last frame.

(reference: loongforge/embodied/data/datasets/video_backends.py:13-154)
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import numpy as np


def _indices_from(timestamps: Sequence[float], fps: float) -> List[int]:
    return [max(0, int(round(float(t) * fps))) for t in timestamps]


def _opencv(path: str, indices, timestamps) -> np.ndarray:
    import cv2

    cap = cv2.VideoCapture(path)
    if not cap.isOpened():
        raise FileNotFoundError(f"cannot open video {path}")
    try:
        n = int(cap.get(cv2.CAP_PROP_FRAME_COUNT))
        if indices is None:
            indices = _indices_from(timestamps, cap.get(cv2.CAP_PROP_FPS) or 30.0)
        want = [min(int(i), max(n - 1, 0)) for i in indices]
        frames: Dict[int, np.ndarray] = {}
        at = -1                                              # index of the frame the next read() returns, once positioned
        for i in sorted(set(want)):
            if at != i:
                cap.set(cv2.CAP_PROP_POS_FRAMES, i)
            ok, fr = cap.read()
            if not ok:
                if not frames:
                    raise IOError(f"no frame {i} in {path}")
                fr = frames[max(frames)][:, :, ::-1]         # a short stream: hold the last frame
            frames[i] = np.ascontiguousarray(fr[:, :, ::-1])
            at = i + 1
        return np.stack([frames[i] for i in want])
    finally:
        cap.release()


def _pyav(path: str, indices, timestamps) -> np.ndarray:
    import av

    with av.open(path) as container:
        stream = container.streams.video[0]
        fps = float(stream.average_rate or 30)
        want = list(indices) if indices is not None else _indices_from(timestamps, fps)
        need, frames = set(want), {}
        for i, frame in enumerate(container.decode(stream)):
            if i in need:
                frames[i] = frame.to_ndarray(format="rgb24")
            if i >= max(need):
                break
        last = frames[max(frames)]
        return np.stack([frames.get(i, last) for i in want])


def _decord(path: str, indices, timestamps) -> np.ndarray:
    import decord

    vr = decord.VideoReader(path)
    want = list(indices) if indices is not None else _indices_from(timestamps, float(vr.get_avg_fps()))
    return vr.get_batch([min(i, len(vr) - 1) for i in want]).asnumpy()


def _torchcodec(path: str, indices, timestamps) -> np.ndarray:
    from torchcodec.decoders import VideoDecoder

    dec = VideoDecoder(path)
    if indices is not None:
        batch = dec.get_frames_at(indices=[min(int(i), len(dec) - 1) for i in indices])
    else:
        batch = dec.get_frames_played_at(seconds=[float(t) for t in timestamps])
    return batch.data.permute(0, 2, 3, 1).contiguous().numpy()


BACKENDS: Dict[str, Callable] = {"opencv": _opencv, "pyav": _pyav, "decord": _decord, "torchcodec": _torchcodec}


def decode_frames(path: str, indices: Optional[Sequence[int]] = None, timestamps: Optional[Sequence[float]] = None,
                  backend: str = "opencv") -> np.ndarray:
    if (indices is None) == (timestamps is None):
        raise ValueError("give exactly one of indices / timestamps")
    if backend not in BACKENDS:
        raise ValueError(f"unknown video backend {backend!r} ({' | '.join(BACKENDS)})")
    try:
        return BACKENDS[backend](path, indices, timestamps)
    except ImportError as e:
        raise ImportError(f"video backend {backend!r} needs a package that is not installed ({e.name}); "
                          f"'opencv' is always available") from e
