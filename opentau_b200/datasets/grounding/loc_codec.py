"""Pixel coordinates <-> PaliGemma ``<locNNNN>`` strings (reference
``src/opentau/datasets/grounding/loc_codec.py:1-330``).

An axis is quantised into 1024 bins of the ORIGINAL image extent: ``bin = clamp(round(coord / extent * 1023))``,
written zero-padded to four digits.  A box is four tokens in ``(y_min, x_min, y_max, x_max)`` order, then a space
and the label; a point is ``(y, x)``; several objects are joined by ``" ; "``.
"""

from __future__ import annotations

import re

NUM_BINS = 1024
MAX_BIN = NUM_BINS - 1
SEGMENT_SEPARATOR = ";"
_LOC = re.compile(r"<loc(\d{4})>")


def _quantize(coord: float, extent: float) -> int:
    if extent <= 0:
        return 0
    return min(MAX_BIN, max(0, int(round(coord / extent * MAX_BIN))))


def _dequantize(bin_idx: int, extent: float) -> float:
    return bin_idx / MAX_BIN * extent


def _tok(b: int) -> str:
    return f"<loc{b:04d}>"


def xyxy_to_loc_tokens(boxes: list[tuple[float, float, float, float]], labels: list[str],
                       image_size: tuple[int, int]) -> str:
    """``boxes`` as ``(x_min, y_min, x_max, y_max)`` pixels, ``image_size = (width, height)``."""
    if len(boxes) != len(labels):
        raise ValueError("boxes and labels differ in length")
    w, h = image_size
    parts = []
    for (x0, y0, x1, y1), label in zip(boxes, labels):
        parts.append(f"{_tok(_quantize(y0, h))}{_tok(_quantize(x0, w))}{_tok(_quantize(y1, h))}{_tok(_quantize(x1, w))} {label}")
    return f" {SEGMENT_SEPARATOR} ".join(parts)


def points_to_loc_tokens(points: list[tuple[float, float]], labels: list[str], image_size: tuple[int, int]) -> str:
    """``points`` as ``(x, y)`` pixels."""
    if len(points) != len(labels):
        raise ValueError("points and labels differ in length")
    w, h = image_size
    return f" {SEGMENT_SEPARATOR} ".join(f"{_tok(_quantize(y, h))}{_tok(_quantize(x, w))} {label}"
                                         for (x, y), label in zip(points, labels))


def _segments(text: str, n: int):
    for seg in text.split(SEGMENT_SEPARATOR):
        bins = [int(b) for b in _LOC.findall(seg)]
        if len(bins) < n:
            continue
        label = _LOC.sub("", seg).strip()
        yield bins[:n], label


def loc_tokens_to_xyxy(text: str, image_size: tuple[int, int]) -> list[tuple[tuple[float, float, float, float], str]]:
    w, h = image_size
    return [((_dequantize(b[1], w), _dequantize(b[0], h), _dequantize(b[3], w), _dequantize(b[2], h)), label)
            for b, label in _segments(text, 4)]


def loc_tokens_to_points(text: str, image_size: tuple[int, int]) -> list[tuple[tuple[float, float], str]]:
    w, h = image_size
    return [((_dequantize(b[1], w), _dequantize(b[0], h)), label) for b, label in _segments(text, 2)]
