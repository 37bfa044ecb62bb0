"""Image augmentation on ``[H, W, C]`` float tensors in ``[0, 1]``: crops, flips, colour and
geometric operations, RandAugment, random erasing, mixup / cutmix.

Covers the role of axlearn/vision/augment.py (the AutoAugment / RandAugment operation table and
policies, ``RandomErasing``) and of the crop / flip preprocessing in axlearn/vision/input_image.py.
Randomness comes from an explicit ``torch.Generator`` so that an input pipeline stays reproducible.
"""

from __future__ import annotations

import math
from typing import Callable, Optional, Sequence

import torch
import torch.nn.functional as F

Tensor = torch.Tensor


def _rand(gen: Optional[torch.Generator]) -> float:
    return float(torch.rand((), generator=gen))


def random_resized_crop(image: Tensor, size: Sequence[int], *, gen=None, scale=(0.08, 1.0), ratio=(3 / 4, 4 / 3)) -> Tensor:
    h, w, _ = image.shape
    for _ in range(10):
        area = h * w * (scale[0] + _rand(gen) * (scale[1] - scale[0]))
        r = math.exp(math.log(ratio[0]) + _rand(gen) * (math.log(ratio[1]) - math.log(ratio[0])))
        ch, cw = int(round(math.sqrt(area / r))), int(round(math.sqrt(area * r)))
        if 0 < ch <= h and 0 < cw <= w:
            top, left = int(_rand(gen) * (h - ch + 1)), int(_rand(gen) * (w - cw + 1))
            return resize(image[top:top + ch, left:left + cw], size)
    return center_crop(image, size)


def resize(image: Tensor, size: Sequence[int]) -> Tensor:
    x = image.permute(2, 0, 1)[None]
    return F.interpolate(x, size=tuple(size), mode="bilinear", align_corners=False, antialias=True)[0].permute(1, 2, 0)


def center_crop(image: Tensor, size: Sequence[int], *, crop_fraction: float = 0.875) -> Tensor:
    h, w, _ = image.shape
    side = int(crop_fraction * min(h, w))
    top, left = (h - side) // 2, (w - side) // 2
    return resize(image[top:top + side, left:left + side], size)


def random_flip(image: Tensor, *, gen=None) -> Tensor:
    return image.flip(1) if _rand(gen) < 0.5 else image


def _blend(a: Tensor, b: Tensor, factor: float) -> Tensor:
    return (a + (b - a) * factor).clamp(0, 1)


def _gray(image: Tensor) -> Tensor:
    return (image * image.new_tensor([0.299, 0.587, 0.114])).sum(-1, keepdim=True).expand_as(image)


def brightness(image, m):
    return _blend(torch.zeros_like(image), image, m)


def color(image, m):
    return _blend(_gray(image), image, m)


def contrast(image, m):
    return _blend(torch.full_like(image, float(_gray(image).mean())), image, m)


def sharpness(image, m):
    k = image.new_tensor([[1, 1, 1], [1, 5, 1], [1, 1, 1]]) / 13
    x = image.permute(2, 0, 1)[:, None]
    blurred = F.conv2d(F.pad(x, (1, 1, 1, 1), mode="replicate"), k[None, None])[:, 0].permute(1, 2, 0)
    return _blend(blurred, image, m)


def posterize(image, bits: int):
    q = 2 ** (8 - int(bits))
    return torch.floor(image * 255 / q) * q / 255


def solarize(image, threshold: float):
    return torch.where(image < threshold, image, 1 - image)


def autocontrast(image, _=None):
    lo, hi = image.amin(dim=(0, 1), keepdim=True), image.amax(dim=(0, 1), keepdim=True)
    return torch.where(hi > lo, (image - lo) / (hi - lo).clamp_min(1e-6), image)


def equalize(image, _=None):
    out = []
    for c in range(image.shape[-1]):
        v = (image[..., c] * 255).round().long().clamp(0, 255)
        hist = torch.bincount(v.reshape(-1), minlength=256).float()
        cdf = hist.cumsum(0)
        nz = cdf[hist > 0]
        if nz.numel() <= 1:
            out.append(image[..., c])
            continue
        lut = ((cdf - nz[0]) / (cdf[-1] - nz[0]).clamp_min(1)).clamp(0, 1)
        out.append(lut[v])
    return torch.stack(out, dim=-1)


def invert(image, _=None):
    return 1 - image


def _affine(image: Tensor, matrix: Sequence[float], fill: float = 0.5) -> Tensor:
    """``matrix = (a, b, tx, c, d, ty)`` maps output pixel offsets from the centre to input offsets."""
    h, w, _ = image.shape
    ys, xs = torch.meshgrid(torch.arange(h, dtype=torch.float32), torch.arange(w, dtype=torch.float32), indexing="ij")
    yc, xc = ys - (h - 1) / 2, xs - (w - 1) / 2
    a, b, tx, c, d, ty = matrix
    sx, sy = a * xc + b * yc + tx + (w - 1) / 2, c * xc + d * yc + ty + (h - 1) / 2
    grid = torch.stack([2 * sx / max(w - 1, 1) - 1, 2 * sy / max(h - 1, 1) - 1], dim=-1)[None]
    x = image.permute(2, 0, 1)[None]
    out = F.grid_sample(x - fill, grid, mode="bilinear", padding_mode="zeros", align_corners=True) + fill
    return out[0].permute(1, 2, 0)


def rotate(image, degrees: float):
    r = math.radians(degrees)
    return _affine(image, (math.cos(r), -math.sin(r), 0, math.sin(r), math.cos(r), 0))


def shear_x(image, m):
    return _affine(image, (1, m, 0, 0, 1, 0))


def shear_y(image, m):
    return _affine(image, (1, 0, 0, m, 1, 0))


def translate_x(image, pixels):
    return _affine(image, (1, 0, pixels, 0, 1, 0))


def translate_y(image, pixels):
    return _affine(image, (1, 0, 0, 0, 1, pixels))


def cutout(image, size: int, *, gen=None, fill: float = 0.5):
    h, w, _ = image.shape
    cy, cx = int(_rand(gen) * h), int(_rand(gen) * w)
    out = image.clone()
    out[max(0, cy - size):cy + size, max(0, cx - size):cx + size] = fill
    return out


# name -> (op, magnitude in [0, 10] -> argument, signed)
_LEVEL = 10.0
_OPS: dict[str, tuple[Callable, Callable[[float], float], bool]] = {
    "AutoContrast": (autocontrast, lambda m: 0, False), "Equalize": (equalize, lambda m: 0, False),
    "Invert": (invert, lambda m: 0, False), "Rotate": (rotate, lambda m: m / _LEVEL * 30, True),
    "Posterize": (posterize, lambda m: 8 - int(m / _LEVEL * 4), False),
    "Solarize": (solarize, lambda m: 1 - m / _LEVEL, False),
    "Color": (color, lambda m: 1 + m / _LEVEL * 0.9, True), "Contrast": (contrast, lambda m: 1 + m / _LEVEL * 0.9, True),
    "Brightness": (brightness, lambda m: 1 + m / _LEVEL * 0.9, True),
    "Sharpness": (sharpness, lambda m: 1 + m / _LEVEL * 0.9, True),
    "ShearX": (shear_x, lambda m: m / _LEVEL * 0.3, True), "ShearY": (shear_y, lambda m: m / _LEVEL * 0.3, True),
    "TranslateX": (translate_x, lambda m: m / _LEVEL * 100, True), "TranslateY": (translate_y, lambda m: m / _LEVEL * 100, True),
}
RANDAUGMENT_OPS = tuple(k for k in _OPS if k != "Invert")


def apply_op(image: Tensor, name: str, magnitude: float, *, gen=None) -> Tensor:
    op, level_fn, signed = _OPS[name]
    arg = level_fn(magnitude)
    if signed and _rand(gen) < 0.5:
        arg = 2 - arg if name in ("Color", "Contrast", "Brightness", "Sharpness") else -arg
    return op(image, arg)


def rand_augment(image: Tensor, *, num_layers: int = 2, magnitude: float = 10.0, gen=None,
                 ops: Sequence[str] = RANDAUGMENT_OPS, prob: float = 1.0) -> Tensor:
    for _ in range(num_layers):
        name = ops[int(_rand(gen) * len(ops)) % len(ops)]
        if _rand(gen) < prob:
            image = apply_op(image, name, magnitude, gen=gen)
    return image


def random_erasing(image: Tensor, *, gen=None, prob: float = 0.25, area=(0.02, 1 / 3), ratio=(0.3, 1 / 0.3)) -> Tensor:
    if _rand(gen) >= prob:
        return image
    h, w, c = image.shape
    for _ in range(10):
        a = h * w * (area[0] + _rand(gen) * (area[1] - area[0]))
        r = math.exp(math.log(ratio[0]) + _rand(gen) * (math.log(ratio[1]) - math.log(ratio[0])))
        eh, ew = int(round(math.sqrt(a * r))), int(round(math.sqrt(a / r)))
        if eh < h and ew < w:
            top, left = int(_rand(gen) * (h - eh)), int(_rand(gen) * (w - ew))
            out = image.clone()
            out[top:top + eh, left:left + ew] = torch.randn(eh, ew, c, generator=gen) * 0.25 + 0.5
            return out.clamp(0, 1)
    return image


def mixup_cutmix(images: Tensor, labels: Tensor, *, num_classes: int, gen=None, mixup_alpha: float = 0.8,
                 cutmix_alpha: float = 1.0, switch_prob: float = 0.5, label_smoothing: float = 0.1):
    """Batch-level mixing; returns mixed ``[B, H, W, C]`` images and soft labels ``[B, classes]``."""
    b, h, w, _ = images.shape
    perm = torch.randperm(b, generator=gen)
    off = label_smoothing / num_classes
    onehot = F.one_hot(labels.long(), num_classes).float() * (1 - label_smoothing) + off
    use_cutmix = cutmix_alpha > 0 and (_rand(gen) < switch_prob or mixup_alpha <= 0)
    alpha = cutmix_alpha if use_cutmix else mixup_alpha
    lam = float(torch.distributions.Beta(alpha, alpha).sample()) if alpha > 0 else 1.0
    if use_cutmix:
        cut = math.sqrt(1 - lam)
        ch, cw = int(h * cut), int(w * cut)
        cy, cx = int(_rand(gen) * h), int(_rand(gen) * w)
        y0, y1, x0, x1 = max(cy - ch // 2, 0), min(cy + ch // 2, h), max(cx - cw // 2, 0), min(cx + cw // 2, w)
        mixed = images.clone()
        mixed[:, y0:y1, x0:x1] = images[perm][:, y0:y1, x0:x1]
        lam = 1 - (y1 - y0) * (x1 - x0) / (h * w)
    else:
        mixed = lam * images + (1 - lam) * images[perm]
    return mixed, lam * onehot + (1 - lam) * onehot[perm]
