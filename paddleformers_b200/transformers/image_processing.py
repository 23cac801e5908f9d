"""Image pre-processing for the vision-language models: dynamic-resolution resize, normalisation and patch extraction in
the order the vision tower expects (roles of paddleformers/transformers/image_processing_utils.py and the Qwen2-VL
image processor of the reference).

``Qwen2VLImageProcessor.__call__(images)`` returns ``pixel_values`` [patches, C * T * P * P] and ``image_grid_thw``
[images, 3]: every image is resized so that both sides are multiples of ``patch_size * merge_size`` with the number of
pixels inside [min_pixels, max_pixels], scaled to [0, 1], normalised, repeated along time to ``temporal_patch_size``
frames, and cut into patches ordered merge-block by merge-block (the 2 x 2 patches that the merger fuses are adjacent).
"""
from __future__ import annotations

import math
from typing import List, Sequence

import numpy as np
import torch

OPENAI_CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
OPENAI_CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280):
    """Target size: both sides multiples of ``factor``, area within the pixel budget, aspect ratio kept as far as the
    rounding allows."""
    if max(height, width) / min(height, width) > 200:
        raise ValueError("aspect ratio above 200 is not supported")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def _resize(img: np.ndarray, h: int, w: int) -> np.ndarray:
    try:
        from PIL import Image

        return np.asarray(Image.fromarray(img).resize((w, h), resample=Image.BICUBIC))
    except ImportError:
        t = torch.from_numpy(img).permute(2, 0, 1)[None].float()
        t = torch.nn.functional.interpolate(t, size=(h, w), mode="bicubic", align_corners=False, antialias=True)
        return t[0].permute(1, 2, 0).round().clamp(0, 255).to(torch.uint8).numpy()


class Qwen2VLImageProcessor:
    def __init__(self, patch_size: int = 14, merge_size: int = 2, temporal_patch_size: int = 2, min_pixels: int = 56 * 56,
                 max_pixels: int = 28 * 28 * 1280, image_mean: Sequence[float] = OPENAI_CLIP_MEAN,
                 image_std: Sequence[float] = OPENAI_CLIP_STD, rescale_factor: float = 1.0 / 255.0, raster_order: bool = False):
        self.patch_size, self.merge_size, self.temporal_patch_size = patch_size, merge_size, temporal_patch_size
        self.raster_order = raster_order           # towers that merge after the encoder read patches row by row (PaddleOCR-VL)
        self.min_pixels, self.max_pixels = min_pixels, max_pixels
        self.mean = np.asarray(image_mean, dtype=np.float32)
        self.std = np.asarray(image_std, dtype=np.float32)
        self.rescale_factor = rescale_factor

    def preprocess_one(self, img: np.ndarray):
        """img: uint8 [H, W, 3]. Returns (patches [grid_h * grid_w, C * T * P * P] float32, (1, grid_h, grid_w))."""
        P, m, T = self.patch_size, self.merge_size, self.temporal_patch_size
        h, w = smart_resize(img.shape[0], img.shape[1], P * m, self.min_pixels, self.max_pixels)
        x = _resize(np.ascontiguousarray(img), h, w).astype(np.float32) * self.rescale_factor
        x = (x - self.mean) / self.std
        x = np.transpose(x, (2, 0, 1))[None].repeat(T, axis=0)               # [T, C, H, W]: a still image fills every frame
        gh, gw = h // P, w // P
        C = x.shape[1]
        if self.raster_order:
            x = x.reshape(T, C, gh, P, gw, P).transpose(2, 4, 1, 0, 3, 5)       # [gh, gw, C, T, P, P]
            return x.reshape(gh * gw, C * T * P * P), (1, gh, gw)
        x = x.reshape(1, T, C, gh // m, m, P, gw // m, m, P)
        x = x.transpose(0, 3, 6, 4, 7, 2, 1, 5, 8)                          # [1, gh/m, gw/m, m, m, C, T, P, P]
        return x.reshape(gh * gw, C * T * P * P), (1, gh, gw)

    def __call__(self, images: List[np.ndarray], return_tensors: str = "pt"):
        patches, grids = zip(*(self.preprocess_one(np.asarray(im)) for im in images))
        pv = np.concatenate(patches, axis=0)
        grid = np.asarray(grids, dtype=np.int64)
        if return_tensors == "pt":
            return {"pixel_values": torch.from_numpy(pv), "image_grid_thw": torch.from_numpy(grid)}
        return {"pixel_values": pv, "image_grid_thw": grid}

    def num_image_tokens(self, grid_thw) -> int:
        t, h, w = (int(v) for v in grid_thw)
        return t * h * w // (self.merge_size ** 2)


class Qwen2VLVideoProcessor(Qwen2VLImageProcessor):
    """Video pre-processing (roles of paddleformers/transformers/video_processing_utils.py and the Qwen2-VL video processor):
    ``__call__(videos)`` takes clips as uint8 arrays [frames, H, W, 3], optionally samples frames uniformly
    (``num_frames`` or ``fps`` with the clip's own ``source_fps``), resizes all frames of a clip to one size whose per-clip
    pixel count (frames x H x W) stays within the budget, pads the clip to a multiple of ``temporal_patch_size`` by repeating
    its last frame, and cuts it into spatio-temporal patches in the tower's merge-block order. Returns
    ``pixel_values_videos`` [patches, C * T * P * P] and ``video_grid_thw`` [clips, 3]."""

    def __init__(self, *args, min_frames: int = 4, max_frames: int = 768, **kw):
        kw.setdefault("min_pixels", 128 * 28 * 28)
        kw.setdefault("max_pixels", 28 * 28 * 768)
        super().__init__(*args, **kw)
        self.min_frames, self.max_frames = min_frames, max_frames

    def sample_indices(self, total: int, num_frames: int = None, fps: float = None, source_fps: float = None) -> np.ndarray:
        """Uniformly spaced frame indices: ``num_frames`` of them, or ``fps`` per second of a clip recorded at ``source_fps``
        (rounded to a multiple of the temporal patch size and clamped to [min_frames, max_frames])."""
        T = self.temporal_patch_size
        if num_frames is None and fps is not None:
            if not source_fps:
                raise ValueError("sampling by fps needs the clip's source_fps")
            n = total / source_fps * fps
            n = min(max(n, self.min_frames), self.max_frames, total)
            num_frames = max(int(math.floor(n / T) * T), T)
        if num_frames is None:
            return np.arange(total)
        if num_frames > total:
            raise ValueError(f"cannot sample {num_frames} frames from a clip of {total}")
        return np.linspace(0, total - 1, num_frames).round().astype(np.int64)

    def preprocess_clip(self, frames: np.ndarray):
        """frames: uint8 [F, H, W, 3] -> (patches [grid_t * grid_h * grid_w, C * T * P * P], (grid_t, grid_h, grid_w))."""
        P, m, T = self.patch_size, self.merge_size, self.temporal_patch_size
        F = frames.shape[0]
        # the pixel budget of a clip is shared by its frames
        h, w = smart_resize(frames.shape[1], frames.shape[2], P * m, self.min_pixels // max(F, 1) if F > 1 else self.min_pixels,
                            max(self.max_pixels // max(F, 1), (P * m) ** 2))
        x = np.stack([_resize(np.ascontiguousarray(f), h, w) for f in frames]).astype(np.float32) * self.rescale_factor
        x = (x - self.mean) / self.std
        x = np.transpose(x, (0, 3, 1, 2))                                    # [F, C, H, W]
        if F % T:
            x = np.concatenate([x, np.repeat(x[-1:], T - F % T, axis=0)], axis=0)
        gt, gh, gw = x.shape[0] // T, h // P, w // P
        C = x.shape[1]
        x = x.reshape(gt, T, C, gh // m, m, P, gw // m, m, P)
        x = x.transpose(0, 3, 6, 4, 7, 2, 1, 5, 8)                          # [gt, gh/m, gw/m, m, m, C, T, P, P]
        return x.reshape(gt * gh * gw, C * T * P * P), (gt, gh, gw)

    def __call__(self, videos: List[np.ndarray], num_frames: int = None, fps: float = None, source_fps=None, return_tensors: str = "pt"):
        patches, grids = [], []
        for i, clip in enumerate(videos):
            clip = np.asarray(clip)
            sf = source_fps[i] if isinstance(source_fps, (list, tuple)) else source_fps
            idx = self.sample_indices(clip.shape[0], num_frames, fps, sf)
            p, g = self.preprocess_clip(clip[idx])
            patches.append(p)
            grids.append(g)
        pv = np.concatenate(patches, axis=0)
        grid = np.asarray(grids, dtype=np.int64)
        if return_tensors == "pt":
            return {"pixel_values_videos": torch.from_numpy(pv), "video_grid_thw": torch.from_numpy(grid)}
        return {"pixel_values_videos": pv, "video_grid_thw": grid}


class SiglipImageProcessor:
    """Fixed-size pre-processing of the SigLIP towers (PaliGemma, Gemma 3, Aya Vision; paddleformers/transformers/paligemma2/
    image_processor.py): every image is resized to ``image_size`` x ``image_size`` (bicubic, antialiased), scaled to [0, 1] and
    normalised. Returns ``pixel_values`` float32 [images, 3, size, size]; each image stands for ``tokens_per_image``
    placeholder tokens."""

    def __init__(self, image_size: int = 224, image_mean=(0.5, 0.5, 0.5), image_std=(0.5, 0.5, 0.5), tokens_per_image: int = 256,
                 rescale_factor: float = 1.0 / 255.0):
        self.image_size, self.tokens_per_image, self.rescale_factor = int(image_size), int(tokens_per_image), rescale_factor
        self.image_mean, self.image_std = tuple(image_mean), tuple(image_std)

    def num_image_tokens(self, grid=None) -> int:
        return self.tokens_per_image

    def __call__(self, images: List[np.ndarray], return_tensors: str = "pt"):
        mean = torch.tensor(self.image_mean, dtype=torch.float32).view(1, 3, 1, 1)
        std = torch.tensor(self.image_std, dtype=torch.float32).view(1, 3, 1, 1)
        out = []
        for img in images:
            t = torch.as_tensor(np.ascontiguousarray(img)).permute(2, 0, 1)[None].float()
            t = torch.nn.functional.interpolate(t, size=(self.image_size, self.image_size), mode="bicubic", align_corners=False,
                                                antialias=True).clamp(0.0, 255.0)
            out.append((t * self.rescale_factor - mean) / std)
        return {"pixel_values": torch.cat(out, dim=0)}


class DynamicHDImageProcessor:
    """Image pre-processing of Phi-4-multimodal (paddleformers/transformers/phi4_multimodal/image_processor.py): the image
    is scaled (keeping its aspect ratio) into a grid of ``crop`` x ``crop`` tiles - as many as it covers, at most ``dynamic_hd``,
    otherwise the grid whose aspect ratio is closest - and padded with white on the right / bottom; a bicubic down-scale of the
    padded picture to one tile is the global view. Returns, per image: ``image_pixel_values`` [1 + tiles, 3, crop, crop] (global
    view first, pixels in [-1, 1]), ``image_attention_mask`` [1 + tiles, crop / patch, crop / patch] (0 on patches that are
    padding only), ``image_sizes`` (height, width of the padded picture) and the number of placeholder tokens the image needs;
    a batch is padded to the largest tile count."""

    def __init__(self, crop: int = 448, patch_size: int = 14, dynamic_hd: int = 36, image_mean=(0.5, 0.5, 0.5), image_std=(0.5, 0.5, 0.5)):
        self.crop, self.patch, self.max_tiles = crop, patch_size, dynamic_hd
        self.mean = torch.tensor(image_mean, dtype=torch.float32).view(3, 1, 1)
        self.std = torch.tensor(image_std, dtype=torch.float32).view(3, 1, 1)

    def grid(self, height: int, width: int):
        """(tile columns, tile rows)."""
        wc, hc = math.ceil(width / self.crop), math.ceil(height / self.crop)
        if wc * hc <= self.max_tiles:
            return wc, hc
        aspect, area = width / height, width * height
        best, best_diff = (1, 1), float("inf")
        cands = sorted({(i, j) for i in range(1, self.max_tiles + 1) for j in range(1, self.max_tiles + 1) if i * j <= self.max_tiles},
                       key=lambda x: x[0] * x[1])
        for i, j in cands:
            diff = abs(aspect - i / j)
            if diff < best_diff:
                best, best_diff = (i, j), diff
            elif diff == best_diff and area > 0.5 * self.crop * self.crop * i * j:
                best = (i, j)                      # a tie goes to the larger grid when the image has the pixels for it
        return best

    def preprocess_one(self, img: np.ndarray):
        S, P = self.crop, self.patch
        t = torch.from_numpy(np.ascontiguousarray(img)).permute(2, 0, 1)             # uint8 [3, H, W]
        H, W = t.shape[-2:]
        wc, hc = self.grid(H, W)
        tw, th = S * wc, S * hc
        if tw / W < th / H:
            nw, nh = tw, int(H * (tw / W))
        else:
            nw, nh = int(W * (th / H)), th
        if min(nw, nh) < 10:
            raise ValueError(f"the aspect ratio is too extreme: scaled size {nw} x {nh}")
        pad_w, pad_h = tw - nw, th - nh
        m = S // P
        mask = torch.ones(m * hc, m * wc)
        if pad_w >= P:
            mask[:, -(pad_w // P):] = 0
        if pad_h >= P:
            mask[-(pad_h // P):, :] = 0
        t = torch.nn.functional.interpolate(t[None], size=(nh, nw), mode="bilinear", antialias=True)[0]
        t = torch.nn.functional.pad(t, (0, pad_w, 0, pad_h), value=255)
        x = (t.float() / 255.0 - self.mean) / self.std
        glob = torch.nn.functional.interpolate(x[None], size=(S, S), mode="bicubic", antialias=False, align_corners=False)[0]
        tiles = x.reshape(3, hc, S, wc, S).permute(1, 3, 0, 2, 4).reshape(hc * wc, 3, S, S)
        tile_masks = mask.reshape(hc, m, wc, m).permute(0, 2, 1, 3).reshape(hc * wc, m, m)
        f = (m + 1) // 2                                                             # pooled patches per tile side
        pooled = tile_masks[:, 0::2, 0::2].reshape(hc, wc, f, f).permute(0, 2, 1, 3).reshape(hc * f, wc * f)
        tokens = f * f + f + 1 + int(pooled.sum()) + int(pooled[:, 0].sum())         # global rows + separators, tiles + row ends
        return torch.cat([glob[None], tiles]), torch.cat([torch.ones(1, m, m), tile_masks]), (th, tw), tokens

    def __call__(self, images: List[np.ndarray], return_tensors: str = "pt"):
        outs = [self.preprocess_one(np.asarray(im)) for im in images]
        n = max(o[0].shape[0] for o in outs)
        pix = torch.stack([torch.cat([o[0], o[0].new_zeros(n - o[0].shape[0], *o[0].shape[1:])]) for o in outs])
        masks = torch.stack([torch.cat([o[1], o[1].new_ones(n - o[1].shape[0], *o[1].shape[1:])]) for o in outs])
        return {"image_pixel_values": pix, "image_attention_mask": masks, "image_sizes": torch.tensor([o[2] for o in outs]),
                "num_img_tokens": [o[3] for o in outs]}


class MolmoImageProcessor:
    """Multi-crop pre-processing of Molmo (paddleformers/transformers/molmo/image_processing.py:45-318). The image is scaled
    and centred (black padding) on a canvas of ``rows x cols`` overlapping crops: neighbouring crops share
    ``overlap_margins`` patches, and every crop contributes only its inner window (plus the outer margin on the border of the
    canvas) to the token grid, so the contributions tile the canvas exactly once. A down-scaled view of the whole image comes
    first. Per image it returns

    * ``images`` [1 + crops, patches, 3 p p]: flattened patches (pixel-major, channel last), CLIP-normalised;
    * ``image_masks`` [1 + crops, patches]: fraction of every patch that shows the image; as in the published pipeline the
      rows belong to the crops in order and a final row of -1 stands for the overview;
    * ``tokens``: start, ``rows`` x (``<im_patch>`` x width, ``<im_col>``), end for the overview, then the same for the canvas
      at pooled (2 x 2 patches) resolution;
    * ``image_input_idx`` [1 + crops, pooled patches per crop]: for every pooled cell of every crop the position of its
      ``<im_patch>`` token inside ``tokens``, or -1 where the cell lies in a margin that the neighbour provides."""

    def __init__(self, max_crops: int = 12, overlap_margins=(4, 4), base_image_input_size=(336, 336), image_token_length_w: int = 12,
                 image_token_length_h: int = 12, image_patch_size: int = 14, image_mean=OPENAI_CLIP_MEAN, image_std=OPENAI_CLIP_STD):
        self.max_crops, self.margins, self.size = max_crops, tuple(overlap_margins), tuple(base_image_input_size)
        self.tw, self.th, self.p = image_token_length_w, image_token_length_h, image_patch_size
        self.mean, self.std = np.asarray(image_mean, dtype=np.float32), np.asarray(image_std, dtype=np.float32)
        assert self.margins[0] % 2 == 0 and self.size[0] == self.size[1]
        assert (self.size[0] // self.p + 1) // 2 == self.th == self.tw, "token grid = crop patches pooled 2 x 2"

    def select_tiling(self, h: int, w: int, window: int) -> tuple:
        """(rows, cols) with rows * cols <= max_crops: the grid that needs the least up-scaling, or, when every grid would
        shrink the image, the one that shrinks it least."""
        cands = sorted(((i, j) for i in range(1, self.max_crops + 1) for j in range(1, self.max_crops + 1) if i * j <= self.max_crops),
                       key=lambda t: (t[0] * t[1], t[0]))
        scale = np.asarray([min(np.float32(i * window) / np.float32(h), np.float32(j * window) / np.float32(w)) for i, j in cands], dtype=np.float32)
        if (scale < 1).all():
            return cands[int(np.argmax(scale))]
        return cands[int(np.argmin(np.where(scale < 1.0, np.float32(10e9), scale)))]

    def resize_and_pad(self, img: np.ndarray, out_hw) -> tuple:
        H, W = out_hw
        h, w = img.shape[:2]
        s = min(np.float32(W) / np.float32(w), np.float32(H) / np.float32(h))
        sh, sw = int(np.float32(h) * s), int(np.float32(w) * s)
        t = torch.from_numpy(np.ascontiguousarray(img)).permute(2, 0, 1).float() / 255.0
        t = torch.nn.functional.interpolate(t[None], size=(sh, sw), mode="bilinear", antialias=True, align_corners=False)[0].clamp(0, 1)
        top, left = (H - sh) // 2, (W - sw) // 2
        canvas = np.zeros((H, W, 3), dtype=np.float32)
        canvas[top:top + sh, left:left + sw] = t.permute(1, 2, 0).numpy()
        mask = np.zeros((H, W), dtype=bool)
        mask[top:top + sh, left:left + sw] = True
        return (canvas - self.mean) / self.std, mask

    def _patchify(self, x: np.ndarray) -> np.ndarray:
        """[n, S, S, c] -> [n, patches, p * p * c] (rows of patches, pixels row by row, channel last)."""
        n, S, _, c = x.shape
        g = S // self.p
        return x.reshape(n, g, self.p, g, self.p, c).transpose(0, 1, 3, 2, 4, 5).reshape(n, g * g, self.p * self.p * c)

    def preprocess_one(self, img: np.ndarray, patch_id: int, col_id: int, start_id: int, end_id: int):
        p, S = self.p, self.size[0]
        lm, rm = self.margins
        g = S // p                                   # patches per crop side
        window = g - (lm + rm)                       # patches that a crop in the middle contributes
        rows, cols = self.select_tiling(img.shape[0] - p * (lm + rm), img.shape[1] - p * (lm + rm), window * p)
        canvas, cmask = self.resize_and_pad(img, (rows * window * p + p * (lm + rm), cols * window * p + p * (lm + rm)))

        def spans(n):                                # per crop along one axis: (first pooled cell used, pooled cells used)
            out = []
            for i in range(n):
                size = window + (lm if i == 0 else 0) + (rm if i == n - 1 else 0)
                out.append((0 if i == 0 else lm // 2, (size + 1) // 2))
            return out

        ys, xs = spans(rows), spans(cols)
        Hp, Wp = (rows * window + lm + rm + 1) // 2, (cols * window + lm + rm + 1) // 2
        assert sum(n for _, n in ys) == Hp and sum(n for _, n in xs) == Wp
        low = [start_id] + ([patch_id] * self.tw + [col_id]) * self.th + [end_id]
        high = [start_id] + ([patch_id] * Wp + [col_id]) * Hp + [end_id]
        tokens = np.asarray(low + high, dtype=np.int64)
        idx = np.full((1 + rows * cols, self.th * self.tw), -1, dtype=np.int64)
        idx[0] = (1 + np.arange(self.th)[:, None] * (self.tw + 1) + np.arange(self.tw)[None]).reshape(-1)
        base = len(low) + 1
        crops, masks, r0 = [], [], 0
        for i, (y0, nh) in enumerate(ys):
            c0 = 0
            for j, (x0, nw) in enumerate(xs):
                cell = np.full((self.th, self.tw), -1, dtype=np.int64)
                cell[y0:y0 + nh, x0:x0 + nw] = base + (r0 + np.arange(nh))[:, None] * (Wp + 1) + (c0 + np.arange(nw))[None]
                idx[1 + i * cols + j] = cell.reshape(-1)
                py, px = i * window * p, j * window * p
                crops.append(canvas[py:py + S, px:px + S])
                masks.append(cmask[py:py + S, px:px + S])
                c0 += nw
            r0 += nh
        whole, _ = self.resize_and_pad(img, self.size)
        images = self._patchify(np.stack([whole] + crops))
        m = self._patchify(np.stack(masks)[..., None].astype(np.float32)).mean(-1)
        image_masks = np.concatenate([m, np.full((1, m.shape[1]), -1.0, dtype=np.float32)], axis=0)
        return images.astype(np.float32), image_masks, tokens, idx
