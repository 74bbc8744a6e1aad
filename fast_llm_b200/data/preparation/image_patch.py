"""Images -> fixed-size patches for the vision encoder.

An image is resized so that both sides are multiples of the patch size (never above the configured maximum, keeping the
aspect ratio), then cut row-major into `[patches, channels, patch_height, patch_width]` with (row, column) coordinates.
In the token stream every patch occupies one placeholder token; optional break / end tokens follow each row / the image.
Parity: `fast_llm/data/preparation/image_patch.py:1-236`.
"""

import io
import math

import numpy as np
import torch


def load_image(image) -> torch.Tensor:
    """bytes / path / PIL image / array -> uint8 [3, height, width]."""
    if torch.is_tensor(image):
        array = image.numpy()
    elif isinstance(image, (np.ndarray, list, tuple)):  # nested lists: arrays that went through a dataset without an Image feature
        array = np.asarray(image, dtype=np.uint8)
    else:
        import PIL.Image

        if isinstance(image, dict) and "bytes" in image:  # the `datasets` Image feature, undecoded
            image = image["bytes"] if image["bytes"] is not None else image["path"]
        if isinstance(image, (bytes, bytearray)):
            image = PIL.Image.open(io.BytesIO(image))
        elif isinstance(image, str):
            image = PIL.Image.open(image)
        array = np.asarray(image.convert("RGB"))
    if array.ndim == 2:
        array = np.repeat(array[:, :, None], 3, axis=2)
    if array.shape[0] != 3 and array.shape[-1] in (1, 3, 4):
        array = array[..., :3] if array.shape[-1] >= 3 else np.repeat(array, 3, axis=-1)
        array = np.transpose(array, (2, 0, 1))
    return torch.from_numpy(np.ascontiguousarray(array)).to(torch.uint8)


def target_size(height: int, width: int, config) -> tuple[int, int]:
    """Largest size with the image's aspect ratio inside the maximum, rounded up to whole patches."""
    ratio = max(height / config.max_image_height, width / config.max_image_width, 1.0)
    height, width = height / ratio, width / ratio
    rows = max(math.ceil(height / config.height - 1e-9), 1)
    columns = max(math.ceil(width / config.width - 1e-9), 1)
    rows = min(rows, config.max_image_height // config.height)
    columns = min(columns, config.max_image_width // config.width)
    return rows * config.height, columns * config.width


def image_to_patches(image, config) -> tuple[torch.Tensor, torch.Tensor, tuple[int, int]]:
    """-> (patches uint8 [rows*columns, 3, ph, pw], coordinates int64 [rows*columns, 2], (rows, columns))."""
    pixels = load_image(image)
    height, width = target_size(pixels.shape[1], pixels.shape[2], config)
    if (height, width) != tuple(pixels.shape[1:]):
        pixels = torch.nn.functional.interpolate(pixels[None].float(), size=(height, width), mode="bicubic", align_corners=False, antialias=True)[0]
        pixels = pixels.round().clamp(0, 255).to(torch.uint8)
    rows, columns = height // config.height, width // config.width
    patches = pixels.reshape(3, rows, config.height, columns, config.width).permute(1, 3, 0, 2, 4).reshape(rows * columns, 3, config.height, config.width)
    coordinates = torch.stack(torch.meshgrid(torch.arange(rows), torch.arange(columns), indexing="ij"), -1).reshape(-1, 2)
    return patches.contiguous(), coordinates, (rows, columns)


def image_token_layout(rows: int, columns: int, config) -> tuple[list[int], list[int]]:
    """Tokens standing for one image and, for every patch (row-major), its index among those tokens."""
    tokens, patch_indices = [], []
    for row in range(rows):
        for _ in range(columns):
            patch_indices.append(len(tokens))
            tokens.append(config.placeholder_token)
        if config.image_break_token is not None and row < rows - 1:
            tokens.append(config.image_break_token)
    if config.image_end_token is not None:
        tokens.append(config.image_end_token)
    return tokens, patch_indices
