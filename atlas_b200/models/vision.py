"""Vision tower (Qwen3.5 / Qwen3-VL style ViT) and the multimodal position bookkeeping (interleaved MRoPE).

An image arrives as flattened patches ``[n_patches, C * Tp * P * P]`` with its grid ``(t, h, w)`` in patches.  The
tower embeds the patches (the 3-D convolution with stride = kernel is a matrix product), adds position embeddings
interpolated bilinearly from a learned square table, runs pre-norm transformer blocks whose attention is full WITHIN a
frame and uses a 2-D rotary embedding (row and column frequencies on the two halves of the rotary dimensions), and
merges each ``m x m`` neighbourhood of patches into one token of the language model's width.  Patches are ordered so
that the ``m x m`` neighbours are consecutive (the processor's order), which is what the merger's reshape relies on.

The language model sees one placeholder token per merged patch; their embeddings are replaced by the tower's output
and their rotary positions are three-dimensional: (time, row, column) offsets from the position where the image
starts, while text tokens advance all three together.  After an image the text continues at
``start + max(rows, columns)``.  The rotary frequencies are dealt to the three position streams round-robin
("interleaved": frequency ``i`` follows the row stream when ``i % 3 == 1`` and ``i < 3 * section[1]``, the column
stream when ``i % 3 == 2`` and ``i < 3 * section[2]``, the time stream otherwise).

The tower runs once per image, outside the token loop, on framework matrix products and attention; the decoder's
hand-written kernels are untouched because MRoPE is presented to them as a step-local rotary table (one row per token)
with ``positions = arange``.

Reference parity: ``crates/spark-model/src/layers/vision/`` (patch embed, blocks, merger), ``kernels/gb10/common/
rope_mrope_interleaved.cu`` (the interleaved frequency assignment), ``crates/spark-server/src/api/multimodal.rs``
(placeholder expansion and position computation).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F


@dataclass
class VisionConfig:
    depth: int = 27
    hidden_size: int = 1152
    intermediate_size: int = 4304
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    out_hidden_size: int = 2048
    num_position_embeddings: int = 2304
    hidden_act: str = "gelu_pytorch_tanh"

    @staticmethod
    def from_hf(d: dict) -> "VisionConfig":
        keys = VisionConfig.__dataclass_fields__.keys()
        return VisionConfig(**{k: d[k] for k in keys if k in d})


class VisionTower:
    def __init__(self, cfg: VisionConfig, device="cpu", dtype=torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.w: Dict[str, torch.Tensor] = {}

    # ------------------------------------------------------------------ weights
    def load(self, get, prefix: str = "model.visual.") -> "VisionTower":
        """``get(name)`` returns a checkpoint tensor; names follow the HF module tree under ``prefix``."""
        c = self.cfg
        names = ["patch_embed.proj.weight", "patch_embed.proj.bias", "pos_embed.weight", "merger.norm.weight", "merger.norm.bias",
                 "merger.linear_fc1.weight", "merger.linear_fc1.bias", "merger.linear_fc2.weight", "merger.linear_fc2.bias"]
        for i in range(c.depth):
            b = f"blocks.{i}."
            names += [b + n for n in ("norm1.weight", "norm1.bias", "norm2.weight", "norm2.bias", "attn.qkv.weight", "attn.qkv.bias",
                                      "attn.proj.weight", "attn.proj.bias", "mlp.linear_fc1.weight", "mlp.linear_fc1.bias",
                                      "mlp.linear_fc2.weight", "mlp.linear_fc2.bias")]
        for n in names:
            self.w[n] = get(prefix + n).to(device=self.device, dtype=self.dtype).contiguous()
        self.w["patch_embed.proj.weight"] = self.w["patch_embed.proj.weight"].reshape(c.hidden_size, -1).contiguous()
        return self

    def init_random(self, seed: int = 0, std: float = 0.02) -> "VisionTower":
        c = self.cfg
        g = torch.Generator().manual_seed(seed)
        r = lambda *s: (torch.randn(*s, generator=g) * std).to(device=self.device, dtype=self.dtype)
        ones = lambda n: torch.ones(n, device=self.device, dtype=self.dtype)
        zeros = lambda n: torch.zeros(n, device=self.device, dtype=self.dtype)
        pd = c.in_channels * c.temporal_patch_size * c.patch_size * c.patch_size
        mh = c.hidden_size * c.spatial_merge_size ** 2
        self.w = {"patch_embed.proj.weight": r(c.hidden_size, pd), "patch_embed.proj.bias": zeros(c.hidden_size),
                  "pos_embed.weight": r(c.num_position_embeddings, c.hidden_size),
                  "merger.norm.weight": ones(c.hidden_size), "merger.norm.bias": zeros(c.hidden_size),
                  "merger.linear_fc1.weight": r(mh, mh), "merger.linear_fc1.bias": zeros(mh),
                  "merger.linear_fc2.weight": r(c.out_hidden_size, mh), "merger.linear_fc2.bias": zeros(c.out_hidden_size)}
        for i in range(c.depth):
            b = f"blocks.{i}."
            self.w.update({b + "norm1.weight": ones(c.hidden_size), b + "norm1.bias": zeros(c.hidden_size),
                           b + "norm2.weight": ones(c.hidden_size), b + "norm2.bias": zeros(c.hidden_size),
                           b + "attn.qkv.weight": r(3 * c.hidden_size, c.hidden_size), b + "attn.qkv.bias": zeros(3 * c.hidden_size),
                           b + "attn.proj.weight": r(c.hidden_size, c.hidden_size), b + "attn.proj.bias": zeros(c.hidden_size),
                           b + "mlp.linear_fc1.weight": r(c.intermediate_size, c.hidden_size),
                           b + "mlp.linear_fc1.bias": zeros(c.intermediate_size),
                           b + "mlp.linear_fc2.weight": r(c.hidden_size, c.intermediate_size),
                           b + "mlp.linear_fc2.bias": zeros(c.hidden_size)})
        return self

    # ------------------------------------------------------------------ position terms
    def _pos_embed(self, grids: Sequence[Tuple[int, int, int]]) -> torch.Tensor:
        """Bilinear interpolation of the learned ``side x side`` table to every grid, in merge-block order."""
        c = self.cfg
        side = int(round(math.sqrt(c.num_position_embeddings)))
        table = self.w["pos_embed.weight"].float()
        m = c.spatial_merge_size
        outs = []
        for t, h, w in grids:
            hi = torch.linspace(0, side - 1, h)
            wi = torch.linspace(0, side - 1, w)
            h0, w0 = hi.floor().long(), wi.floor().long()
            h1, w1 = (h0 + 1).clamp(max=side - 1), (w0 + 1).clamp(max=side - 1)
            dh, dw = (hi - h0)[:, None], (wi - w0)[None, :]
            idx = lambda a, b: (a[:, None] * side + b[None, :]).reshape(-1).to(table.device)
            wgt = lambda x: x.reshape(-1, 1).to(table.device)
            pe = (table[idx(h0, w0)] * wgt((1 - dh) * (1 - dw)) + table[idx(h0, w1)] * wgt((1 - dh) * dw)
                  + table[idx(h1, w0)] * wgt(dh * (1 - dw)) + table[idx(h1, w1)] * wgt(dh * dw))        # [h*w, C] row-major
            pe = pe.view(h // m, m, w // m, m, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)
            outs.append(pe.repeat(t, 1))
        return torch.cat(outs).to(self.dtype)

    def _rotary(self, grids: Sequence[Tuple[int, int, int]]) -> Tuple[torch.Tensor, torch.Tensor]:
        c = self.cfg
        hd = c.hidden_size // c.num_heads
        quarter = hd // 4                                     # frequencies per axis (row / column)
        inv = 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2, dtype=torch.float32) / (hd // 2)))
        m = c.spatial_merge_size
        rows, cols = [], []
        for t, h, w in grids:
            r = torch.arange(h).view(h // m, 1, m, 1).expand(h // m, w // m, m, m).reshape(-1)
            cc = torch.arange(w).view(1, w // m, 1, m).expand(h // m, w // m, m, m).reshape(-1)
            rows.append(r.repeat(t))
            cols.append(cc.repeat(t))
        r, cc = torch.cat(rows).float(), torch.cat(cols).float()
        ang = torch.cat([r[:, None] * inv[None, :quarter], cc[:, None] * inv[None, :quarter]], -1)     # [N, hd/2]
        emb = torch.cat([ang, ang], -1).to(self.device)
        return emb.cos(), emb.sin()

    # ------------------------------------------------------------------ forward
    @torch.inference_mode()
    def forward(self, patches: torch.Tensor, grids: Sequence[Tuple[int, int, int]]) -> torch.Tensor:
        """``patches [sum(t*h*w), C*Tp*P*P]`` in the processor's merge-block order -> ``[sum(t*h*w) / m^2, out_hidden]``."""
        c, w = self.cfg, self.w
        H, nh = c.hidden_size, c.num_heads
        hd = H // nh
        x = F.linear(patches.to(device=self.device, dtype=self.dtype), w["patch_embed.proj.weight"], w["patch_embed.proj.bias"])
        x = x + self._pos_embed(grids)
        cos, sin = self._rotary(grids)
        cos, sin = cos[:, None, :], sin[:, None, :]
        bounds = [0]
        for t, h, ww in grids:
            for _ in range(t):
                bounds.append(bounds[-1] + h * ww)
        act = (lambda v: F.gelu(v, approximate="tanh")) if c.hidden_act == "gelu_pytorch_tanh" else F.gelu

        def rot(v):
            vf = v.float()
            half = vf.shape[-1] // 2
            r = torch.cat([-vf[..., half:], vf[..., :half]], -1)
            return (vf * cos + r * sin).to(v.dtype)

        for i in range(c.depth):
            b = f"blocks.{i}."
            h1 = F.layer_norm(x, (H,), w[b + "norm1.weight"], w[b + "norm1.bias"], 1e-6)
            qkv = F.linear(h1, w[b + "attn.qkv.weight"], w[b + "attn.qkv.bias"]).view(-1, 3, nh, hd)
            q, k, v = rot(qkv[:, 0]), rot(qkv[:, 1]), qkv[:, 2]
            outs = []
            for lo, hi in zip(bounds[:-1], bounds[1:]):                     # full attention inside one frame
                o = F.scaled_dot_product_attention(q[lo:hi].transpose(0, 1)[None], k[lo:hi].transpose(0, 1)[None],
                                                   v[lo:hi].transpose(0, 1)[None])
                outs.append(o[0].transpose(0, 1).reshape(hi - lo, H))
            x = x + F.linear(torch.cat(outs), w[b + "attn.proj.weight"], w[b + "attn.proj.bias"])
            h2 = F.layer_norm(x, (H,), w[b + "norm2.weight"], w[b + "norm2.bias"], 1e-6)
            x = x + F.linear(act(F.linear(h2, w[b + "mlp.linear_fc1.weight"], w[b + "mlp.linear_fc1.bias"])),
                             w[b + "mlp.linear_fc2.weight"], w[b + "mlp.linear_fc2.bias"])
        x = F.layer_norm(x, (H,), w["merger.norm.weight"], w["merger.norm.bias"], 1e-6).view(-1, H * c.spatial_merge_size ** 2)
        x = F.linear(F.gelu(F.linear(x, w["merger.linear_fc1.weight"], w["merger.linear_fc1.bias"])),
                     w["merger.linear_fc2.weight"], w["merger.linear_fc2.bias"])
        return x


# ----------------------------------------------------------------------------- image -> patches
def patchify(image: np.ndarray, cfg: VisionConfig, mean=(0.5, 0.5, 0.5), std=(0.5, 0.5, 0.5),
             max_pixels: int = 1280 * 28 * 28) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
    """``image [H, W, 3]`` uint8 -> (patches ``[h*w, C*Tp*P*P]`` in merge-block order, grid ``(1, h, w)``).  The image is
    resized so both sides are multiples of ``patch * merge`` (and the area stays under ``max_pixels``), normalised,
    repeated along time to fill a temporal patch."""
    P, m, Tp = cfg.patch_size, cfg.spatial_merge_size, cfg.temporal_patch_size
    unit = P * m
    H0, W0 = image.shape[:2]
    scale = min(1.0, math.sqrt(max_pixels / max(1, H0 * W0)))
    Hn, Wn = max(unit, int(round(H0 * scale / unit)) * unit), max(unit, int(round(W0 * scale / unit)) * unit)
    x = torch.from_numpy(np.array(image, dtype=np.uint8)).permute(2, 0, 1).float()[None] / 255.0
    if (Hn, Wn) != (H0, W0):
        x = F.interpolate(x, size=(Hn, Wn), mode="bilinear", align_corners=False, antialias=True)
    x = (x[0] - torch.tensor(mean).view(3, 1, 1)) / torch.tensor(std).view(3, 1, 1)
    h, w = Hn // P, Wn // P
    x = x[:, None].expand(3, Tp, Hn, Wn)                                     # [C, Tp, H, W]
    x = x.reshape(3, Tp, h // m, m, P, w // m, m, P).permute(2, 5, 3, 6, 0, 1, 4, 7)      # [h/m, w/m, m, m, C, Tp, P, P]
    return x.reshape(h * w, 3 * Tp * P * P).contiguous(), (1, h, w)


# ----------------------------------------------------------------------------- positions
def mrope_positions(token_ids: Sequence[int], image_token_id: int, grids: Sequence[Tuple[int, int, int]], merge: int,
                    ) -> Tuple[np.ndarray, int]:
    """Three position streams ``[3, len(token_ids)]`` (time, row, column) and the offset ``delta`` such that a token
    generated at index ``i`` sits at position ``i + delta`` on all three.  Each run of image placeholders consumes the
    next grid."""
    n = len(token_ids)
    pos = np.zeros((3, n), dtype=np.int64)
    cur, i, gi = 0, 0, 0
    while i < n:
        if token_ids[i] != image_token_id:
            pos[:, i] = cur
            cur += 1
            i += 1
            continue
        t, h, w = grids[gi]
        gi += 1
        gh, gw = h // merge, w // merge
        cnt = t * gh * gw
        if i + cnt > n or any(tok != image_token_id for tok in token_ids[i:i + cnt]):
            raise ValueError("image placeholder run does not match its grid")
        pos[0, i:i + cnt] = cur
        pos[1, i:i + cnt] = cur + np.repeat(np.arange(gh), gw * t)
        pos[2, i:i + cnt] = cur + np.tile(np.arange(gw), gh * t)
        cur += max(gh, gw)
        i += cnt
    if gi != len(grids):
        raise ValueError("more images than placeholder runs")
    return pos, int(cur - n)


def mrope_table(rope_cache: torch.Tensor, positions3: torch.Tensor, section: Sequence[int]) -> torch.Tensor:
    """Step-local rotary table ``[T, rotary_dim]`` (first half cos, second half sin) for three position streams
    ``positions3 [3, T]``: frequency ``i`` reads the row of the stream it is dealt to."""
    half = rope_cache.shape[1] // 2
    i = torch.arange(half, device=rope_cache.device)
    stream = torch.zeros(half, dtype=torch.long, device=rope_cache.device)
    stream[(i % 3 == 1) & (i < 3 * section[1])] = 1
    stream[(i % 3 == 2) & (i < 3 * section[2])] = 2
    p = positions3.long()[stream]                            # [half, T]: position each frequency uses
    cols = i[:, None].expand_as(p)
    cos = rope_cache[p, cols]
    sin = rope_cache[p, cols + half]
    return torch.cat([cos.t(), sin.t()], -1).contiguous()


@dataclass
class MultiModalInputs:
    """Per-request multimodal state kept on the sequence."""
    embeds: torch.Tensor                  # [n_placeholders, hidden]: tower output in prompt order
    index_of: np.ndarray                  # [prompt_len]: row of ``embeds`` for a placeholder position, -1 for text
    positions3: np.ndarray                # [3, prompt_len]
    delta: int

    def positions(self, lo: int, hi: int) -> np.ndarray:
        n = self.positions3.shape[1]
        out = np.empty((3, hi - lo), dtype=np.int64)
        a, b = min(lo, n), min(hi, n)
        out[:, :b - a] = self.positions3[:, a:b]
        if hi > n:
            out[:, b - a:] = np.arange(max(lo, n), hi)[None, :] + self.delta
        return out


def prepare(tower: VisionTower, token_ids: Sequence[int], image_token_id: int, images: Sequence[Tuple[torch.Tensor, Tuple[int, int, int]]],
            ) -> MultiModalInputs:
    """Runs the tower over the request's images (``(patches, grid)`` pairs) and lays out placeholders and positions."""
    grids = [g for _, g in images]
    embeds = tower.forward(torch.cat([p for p, _ in images]), grids)
    pos3, delta = mrope_positions(token_ids, image_token_id, grids, tower.cfg.spatial_merge_size)
    is_img = np.asarray([t == image_token_id for t in token_ids])
    if int(is_img.sum()) != embeds.shape[0]:
        raise ValueError(f"{int(is_img.sum())} image placeholders but the tower produced {embeds.shape[0]} tokens")
    index_of = np.where(is_img, np.cumsum(is_img) - 1, -1)
    return MultiModalInputs(embeds, index_of, pos3, delta)
