"""Image input: decode -> smart resize -> bicubic antialias resample (uint8) -> rescale + normalise
(fp32) -> temporal duplicate -> patch rows `pixel_values [L, 1536]` in spatial-merge order and
`grid_thw = (1, H'/16, W'/16)`; plus the prompt-side helpers: `<|image_pad|>` expansion and the
three-axis rotary positions of a prompt with images.

Parity: `crates/saber-vision-input/src/processor.rs:1-120` (processor constants, `smart_resize` in
double precision with round-half-even), `src/resize.rs` (separable bicubic with antialiasing on
uint8), `src/decode.rs` / `src/exif.rs` (decode + EXIF orientation), `src/url.rs` (data URLs).
"""
from __future__ import annotations

import base64
import io
import math
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np


class ImageInputError(ValueError):
    """A request-level (HTTP 400) problem with an image."""


@dataclass(frozen=True)
class ProcessorConfig:
    patch_size: int = 16
    temporal_patch_size: int = 2
    merge_size: int = 2
    min_pixels: int = 65_536
    max_pixels: int = 16_777_216
    image_mean: tuple = (0.5, 0.5, 0.5)
    image_std: tuple = (0.5, 0.5, 0.5)
    rescale_factor: float = 1.0 / 255.0

    @property
    def factor(self) -> int:
        return self.patch_size * self.merge_size

    @property
    def row_len(self) -> int:
        return 3 * self.temporal_patch_size * self.patch_size * self.patch_size

    def clamped_to_arena(self, arena_patches: int) -> "ProcessorConfig":
        """The same processor with its pixel ceiling lowered to what a tower arena of
        `arena_patches` patch rows holds (0 = no clamp): larger images are downscaled, not refused."""
        if arena_patches <= 0:
            return self
        cap = min(self.max_pixels, arena_patches * self.patch_size * self.patch_size)
        return ProcessorConfig(self.patch_size, self.temporal_patch_size, self.merge_size, self.min_pixels,
                               cap, self.image_mean, self.image_std, self.rescale_factor)


def smart_resize(height: int, width: int, factor: int = 32, min_pixels: int = 65_536,
                 max_pixels: int = 16_777_216) -> tuple:
    """Target (H', W'): both multiples of `factor`, pixel count inside [min, max], aspect kept."""
    if height <= 0 or width <= 0:
        raise ImageInputError("image has no pixels")
    ratio = max(height, width) / min(height, width)
    if ratio > 200:
        raise ImageInputError(f"absolute aspect ratio must be smaller than 200, got {ratio!r}")
    h_bar = round(height / factor) * factor          # Python's round: ties to even
    w_bar = round(width / factor) * factor
    if h_bar * w_bar > max_pixels:
        beta = math.sqrt((height * width) / max_pixels)
        h_bar = max(factor, math.floor(height / beta / factor) * factor)
        w_bar = max(factor, math.floor(width / beta / factor) * factor)
    elif h_bar * w_bar < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h_bar = math.ceil(height * beta / factor) * factor
        w_bar = math.ceil(width * beta / factor) * factor
    return int(h_bar), int(w_bar)


# ----------------------------------------------------------------------------------- resample
def _cubic(x: np.ndarray, a: float = -0.5) -> np.ndarray:
    x = np.abs(x)
    return np.where(x < 1.0, ((a + 2.0) * x - (a + 3.0)) * x * x + 1.0,
                    np.where(x < 2.0, (((x - 5.0) * x + 8.0) * x - 4.0) * a, 0.0))


def _axis_weights(n_in: int, n_out: int):
    """Per output index: first input index and the normalised filter taps (antialiased bicubic: the
    kernel's support is stretched by the downscale factor)."""
    scale = n_in / n_out
    support = 2.0 * max(scale, 1.0)
    inv = 1.0 / max(scale, 1.0)
    starts, taps = [], []
    for i in range(n_out):
        center = scale * (i + 0.5)
        lo = max(int(center - support + 0.5), 0)
        hi = min(int(center + support + 0.5), n_in)
        xs = np.arange(lo, hi, dtype=np.float64)
        w = _cubic((xs - center + 0.5) * inv)
        s = w.sum()
        starts.append(lo)
        taps.append(w / s if s != 0 else w)
    return starts, taps


def resample_bicubic_aa_np(img: np.ndarray, size: tuple) -> np.ndarray:
    """uint8 [H, W, C] -> uint8 [H', W', C]: separable antialiased bicubic (a = -0.5), horizontal
    pass then vertical, each rounded to uint8 (the CPU restatement; `resize` uses torch's kernel)."""
    H, W, _ = img.shape
    Ho, Wo = size
    x = img.astype(np.float64)
    starts, taps = _axis_weights(W, Wo)
    tmp = np.empty((H, Wo, img.shape[2]))
    for j in range(Wo):
        tmp[:, j] = np.tensordot(x[:, starts[j]:starts[j] + len(taps[j])], taps[j], axes=([1], [0]))
    tmp = np.clip(np.floor(tmp + 0.5), 0, 255)
    starts, taps = _axis_weights(H, Ho)
    out = np.empty((Ho, Wo, img.shape[2]))
    for i in range(Ho):
        out[i] = np.tensordot(taps[i], tmp[starts[i]:starts[i] + len(taps[i])], axes=([0], [0]))
    return np.clip(np.floor(out + 0.5), 0, 255).astype(np.uint8)


def resize(img: np.ndarray, size: tuple) -> np.ndarray:
    """uint8 [H, W, 3] -> uint8 [H', W', 3] with torch's antialiased bicubic kernel on uint8."""
    if tuple(img.shape[:2]) == tuple(size):
        return img
    import torch
    import torch.nn.functional as TF
    x = torch.from_numpy(np.array(img, dtype=np.uint8, order="C")).permute(2, 0, 1)[None]   # (a copy: decoded images are read-only views)
    try:
        y = TF.interpolate(x, size=tuple(size), mode="bicubic", antialias=True, align_corners=False)
    except (RuntimeError, NotImplementedError):
        y = TF.interpolate(x.float(), size=tuple(size), mode="bicubic", antialias=True, align_corners=False)
        y = y.round().clamp(0, 255).to(torch.uint8)
    return y[0].permute(1, 2, 0).contiguous().numpy()


# ----------------------------------------------------------------------------------- patch rows
@dataclass
class Processed:
    pixel_values: np.ndarray      # fp32 [L, row_len], spatial-merge order
    grid_thw: tuple               # (1, H'/p, W'/p)
    resized_hw: tuple

    @property
    def patches(self) -> int:
        return self.pixel_values.shape[0]

    def merged_tokens(self, merge: int = 2) -> int:
        return self.patches // (merge * merge)


def patchify(norm: np.ndarray, cfg: ProcessorConfig) -> np.ndarray:
    """fp32 [3, H', W'] -> [L, 3 * T * p * p]; rows ordered (H'/pm, W'/pm, m, m), a row (C, T, p, p)."""
    C, H, W = norm.shape
    p, m, T = cfg.patch_size, cfg.merge_size, cfg.temporal_patch_size
    gh, gw = H // p, W // p
    x = np.broadcast_to(norm[None], (T, C, H, W))
    x = x.reshape(T, C, gh // m, m, p, gw // m, m, p)
    x = x.transpose(2, 5, 3, 6, 1, 0, 4, 7)           # gh/m, gw/m, m, m, C, T, p, p
    return np.ascontiguousarray(x).reshape(gh * gw, C * T * p * p).astype(np.float32)


def process_image(img: np.ndarray, cfg: ProcessorConfig = ProcessorConfig()) -> Processed:
    """RGB uint8 [H, W, 3] -> patch rows."""
    if img.ndim != 3 or img.shape[2] != 3 or img.dtype != np.uint8:
        raise ImageInputError("expected an RGB uint8 image [H, W, 3]")
    Ht, Wt = smart_resize(img.shape[0], img.shape[1], cfg.factor, cfg.min_pixels, cfg.max_pixels)
    r = resize(img, (Ht, Wt))
    mean = np.asarray(cfg.image_mean, dtype=np.float32)
    std = np.asarray(cfg.image_std, dtype=np.float32)
    # rescale and normalise fused: x * (rescale / std) - mean / std, in fp32
    norm = r.astype(np.float32) * (np.float32(cfg.rescale_factor) / std) - mean / std
    norm = norm.transpose(2, 0, 1)
    return Processed(patchify(norm, cfg), (1, Ht // cfg.patch_size, Wt // cfg.patch_size), (Ht, Wt))


# ----------------------------------------------------------------------------------- decode, URLs
def decode_image(data: bytes) -> np.ndarray:
    """JPEG / PNG / WebP bytes -> RGB uint8 [H, W, 3], EXIF orientation applied."""
    try:
        from PIL import Image, ImageOps
    except ImportError as e:                                   # pragma: no cover
        raise ImageInputError("image decoding needs Pillow") from e
    try:
        im = Image.open(io.BytesIO(data))
        im = ImageOps.exif_transpose(im)
        if im.mode in ("RGBA", "LA", "P"):                     # composite transparency over white
            im = im.convert("RGBA")
            bg = Image.new("RGBA", im.size, (255, 255, 255, 255))
            im = Image.alpha_composite(bg, im)
        im = im.convert("RGB")
    except ImageInputError:
        raise
    except Exception as e:
        raise ImageInputError(f"cannot decode image: {e}") from e
    return np.asarray(im, dtype=np.uint8)


def fetch_image_url(url: str, allow_files: bool = False, max_bytes: int = 64 << 20) -> bytes:
    """`data:` URLs (base64 or percent-encoded) always; `file://` only when the operator allows it;
    network URLs are refused (the server makes no outbound requests)."""
    if url.startswith("data:"):
        head, sep, body = url.partition(",")
        if not sep:
            raise ImageInputError("malformed data URL")
        if head.endswith(";base64"):
            try:
                raw = base64.b64decode(body, validate=False)
            except Exception as e:
                raise ImageInputError(f"malformed base64 in data URL: {e}") from e
        else:
            from urllib.parse import unquote_to_bytes
            raw = unquote_to_bytes(body)
    elif url.startswith("file://"):
        if not allow_files:
            raise ImageInputError("file URLs are disabled")
        with open(url[len("file://"):], "rb") as f:
            raw = f.read(max_bytes + 1)
    else:
        raise ImageInputError("only data: URLs are accepted (this server makes no outbound requests)")
    if len(raw) > max_bytes:
        raise ImageInputError("image too large")
    return raw


# ----------------------------------------------------------------------------------- prompt side
def expand_image_pads(token_ids: Sequence[int], image_pad_id: int, grids: Sequence[tuple],
                      merge: int = 2) -> list:
    """Every `<|image_pad|>` placeholder becomes t * h * w / merge^2 copies, in order of appearance."""
    out, k = [], 0
    for t in token_ids:
        if t == image_pad_id:
            if k >= len(grids):
                raise ImageInputError("more image placeholders than images")
            g = grids[k]
            out.extend([image_pad_id] * (g[0] * g[1] * g[2] // (merge * merge)))
            k += 1
        else:
            out.append(t)
    if k != len(grids):
        raise ImageInputError("more images than image placeholders")
    return out


def mrope_positions(token_ids: Sequence[int], image_pad_id: int, grids: Sequence[tuple], merge: int = 2):
    """Three-axis rotary positions of an EXPANDED prompt: text tokens advance all three axes together;
    an image span of (t, h/m, w/m) tokens starting at s takes (s + ti, s + row, s + col); the text
    after it resumes at max + 1.  Returns (int32 [3, N], delta) with delta = next position - N, the
    offset every later (generated) token adds to its index."""
    n = len(token_ids)
    pos = np.zeros((3, n), dtype=np.int32)
    i, nxt, k = 0, 0, 0
    while i < n:
        if token_ids[i] != image_pad_id:
            pos[:, i] = nxt
            nxt += 1
            i += 1
            continue
        if k >= len(grids):
            raise ImageInputError("more image spans than images")
        t, h, w = grids[k]
        gh, gw = h // merge, w // merge
        span = t * gh * gw
        if i + span > n or any(x != image_pad_id for x in token_ids[i:i + span]):
            raise ImageInputError("image span shorter than its grid")
        ti, r, c = np.meshgrid(np.arange(t), np.arange(gh), np.arange(gw), indexing="ij")
        pos[0, i:i + span] = nxt + ti.reshape(-1)
        pos[1, i:i + span] = nxt + r.reshape(-1)
        pos[2, i:i + span] = nxt + c.reshape(-1)
        nxt += max(t, gh, gw)
        i += span
        k += 1
    return pos, int(nxt - n)
