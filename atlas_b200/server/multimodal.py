"""Image inputs of chat requests: decode the pixel data of ``image_url`` / ``image`` / ``input_image`` content parts,
cut it into the vision tower's patches and widen each image placeholder of the rendered prompt to one token per
merged patch.

Accepted sources: ``data:image/...;base64,...`` URLs, bare base64 strings, Anthropic-style ``{"source": {"type":
"base64", "data": ...}}`` parts and local ``file://`` paths.  Remote URLs are refused (the server does not fetch).

Reference parity: ``crates/spark-server/src/api/multimodal.rs`` (content-part decoding, placeholder expansion).
"""
from __future__ import annotations

import base64
import io
from typing import Any, Dict, List, Sequence, Tuple

import numpy as np


class ImageError(ValueError):
    pass


def _decode(data: bytes) -> np.ndarray:
    try:
        from PIL import Image
    except ImportError as e:                                   # pragma: no cover
        raise ImageError("image inputs need the Pillow package") from e
    try:
        img = Image.open(io.BytesIO(data)).convert("RGB")
    except Exception as e:
        raise ImageError(f"could not decode the image: {e}") from e
    return np.asarray(img, dtype=np.uint8)


def _from_ref(ref: str) -> np.ndarray:
    if ref.startswith("data:"):
        head, _, payload = ref.partition(",")
        if ";base64" not in head:
            raise ImageError("data URLs must be base64 encoded")
        return _decode(base64.b64decode(payload))
    if ref.startswith("file://"):
        with open(ref[len("file://"):], "rb") as f:
            return _decode(f.read())
    if ref.startswith(("http://", "https://")):
        raise ImageError("remote image URLs are not fetched; send the image as a data URL")
    try:
        return _decode(base64.b64decode(ref, validate=True))
    except ImageError:
        raise
    except Exception as e:
        raise ImageError("unrecognised image reference") from e


def extract_images(messages: Sequence[Dict[str, Any]]) -> List[np.ndarray]:
    """Images of all content parts, in prompt order (the order their placeholders are rendered in)."""
    out: List[np.ndarray] = []
    for m in messages:
        c = m.get("content")
        if not isinstance(c, list):
            continue
        for p in c:
            t = p.get("type")
            if t == "image_url":
                u = p.get("image_url")
                out.append(_from_ref(u.get("url", "") if isinstance(u, dict) else str(u)))
            elif t in ("image", "input_image"):
                src = p.get("source") or {}
                if src.get("type") == "base64" and src.get("data"):
                    out.append(_decode(base64.b64decode(src["data"])))
                elif p.get("image_url"):
                    u = p["image_url"]
                    out.append(_from_ref(u.get("url", "") if isinstance(u, dict) else str(u)))
                elif p.get("data"):
                    out.append(_from_ref(str(p["data"])))
                else:
                    raise ImageError("image part without data")
    return out


def expand_placeholders(tokens: Sequence[int], image_token_id: int, counts: Sequence[int]) -> List[int]:
    """Every single image placeholder becomes ``counts[i]`` of them (one per merged patch of image ``i``)."""
    out: List[int] = []
    i = 0
    for t in tokens:
        if t == image_token_id:
            if i >= len(counts):
                raise ImageError("the prompt has more image placeholders than images")
            out.extend([t] * counts[i])
            i += 1
        else:
            out.append(t)
    if i != len(counts):
        raise ImageError(f"{len(counts)} images but {i} placeholders in the rendered prompt")
    return out


def prepare_images(messages, tokens: Sequence[int], vision_cfg, image_token_id: int) -> Tuple[List[int], List[tuple]]:
    """(tokens with widened placeholders, ``(patches, grid)`` per image) for ``LLMEngine.add_request(images=...)``."""
    from ..models.vision import patchify
    imgs = extract_images(messages)
    if not imgs:
        return list(tokens), []
    pairs = [patchify(im, vision_cfg) for im in imgs]
    m2 = vision_cfg.spatial_merge_size ** 2
    counts = [g[0] * g[1] * g[2] // m2 for _, g in pairs]
    return expand_placeholders(tokens, image_token_id, counts), pairs
