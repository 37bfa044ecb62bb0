"""Drawing detections onto images (reference: axlearn/vision/utils_visualization.py:12-110).
Pure numpy on ``uint8 [H, W, 3]`` arrays; ``write_ppm`` stores a result without any image library."""

from __future__ import annotations

from typing import Optional, Sequence

import numpy as np

_PALETTE = np.asarray([[230, 25, 75], [60, 180, 75], [255, 225, 25], [0, 130, 200], [245, 130, 48], [145, 30, 180],
                       [70, 240, 240], [240, 50, 230], [210, 245, 60], [250, 190, 190]], dtype=np.uint8)


def draw_box_on_image(image: np.ndarray, box: Sequence[float], *, color: Sequence[int] = (255, 0, 0),
                      thickness: int = 2, normalized: bool = False) -> np.ndarray:
    """Draws the outline of ``box`` (``ymin, xmin, ymax, xmax``; pixels, or fractions of the image
    when ``normalized``) in place and returns the image.  Parts outside the image are clipped."""
    h, w = image.shape[:2]
    y0, x0, y1, x1 = (float(v) for v in box)
    if normalized:
        y0, x0, y1, x1 = y0 * h, x0 * w, y1 * h, x1 * w
    y0, x0 = int(np.clip(round(y0), 0, h - 1)), int(np.clip(round(x0), 0, w - 1))
    y1, x1 = int(np.clip(round(y1), 0, h - 1)), int(np.clip(round(x1), 0, w - 1))
    if y1 < y0 or x1 < x0:
        return image
    t = max(1, int(thickness))
    c = np.asarray(color, dtype=image.dtype)
    image[y0:min(y0 + t, y1 + 1), x0:x1 + 1] = c
    image[max(y1 - t + 1, y0):y1 + 1, x0:x1 + 1] = c
    image[y0:y1 + 1, x0:min(x0 + t, x1 + 1)] = c
    image[y0:y1 + 1, max(x1 - t + 1, x0):x1 + 1] = c
    return image


def visualize_detections(images: np.ndarray, *, boxes: np.ndarray, scores: np.ndarray, classes: np.ndarray,
                         num_detections: Optional[np.ndarray] = None, min_score_thresh: float = 0.3,
                         max_boxes_to_draw: int = 20, thickness: int = 2) -> np.ndarray:
    """``images [B, H, W, 3]`` uint8 with the (score-sorted) detections above the threshold drawn,
    one colour per class.  ``boxes [B, N, 4]`` in pixels; padded entries have class < 0 or lie
    beyond ``num_detections``."""
    out = np.array(images, dtype=np.uint8, copy=True)
    for b in range(out.shape[0]):
        n = boxes.shape[1] if num_detections is None else int(num_detections[b])
        order = np.argsort(-scores[b, :n], kind="stable")[:max_boxes_to_draw]
        for i in order:
            if scores[b, i] < min_score_thresh or classes[b, i] < 0:
                continue
            draw_box_on_image(out[b], boxes[b, i], color=_PALETTE[int(classes[b, i]) % len(_PALETTE)],
                              thickness=thickness)
    return out


def write_ppm(path: str, image: np.ndarray) -> None:
    """Binary PPM (P6) of a ``uint8 [H, W, 3]`` image."""
    h, w = image.shape[:2]
    with open(path, "wb") as f:
        f.write(f"P6\n{w} {h}\n255\n".encode())
        f.write(np.ascontiguousarray(image, dtype=np.uint8).tobytes())
