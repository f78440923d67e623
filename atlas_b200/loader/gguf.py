"""GGUF container: reader, block de-quantisers and the mapping onto this engine's decoder.

A GGUF file is ``magic | version | n_tensors | n_kv | metadata key/values | tensor infos | padding | tensor data``.
Tensor data is stored in ggml block formats; the ones read here are F32, F16, BF16, Q8_0, Q4_0, Q4_1, Q5_0, Q4_K,
Q5_K, Q6_K (K-quants use 256-element super-blocks with 6-bit sub-block scales).  Weights are de-quantised to the model
dtype at load (and may then be re-quantised to FP8 block scale / NVFP4 by the usual loader path), so every GEMM kernel
of the engine applies unchanged.

``llama``-architecture files store q/k projection rows permuted for ggml's interleaved rotary layout; they are permuted
back to the half-split layout the engine's RoPE kernel uses.  ``qwen2`` / ``qwen3`` files need no permutation.

Reference parity: ``crates/spark-runtime/src/weights/gguf.rs`` (container + K-quant decode),
``crates/avarok-core/src/config/gguf.rs:83-92`` (architecture -> loader mapping: llama / qwen2 -> GQA + SwiGLU,
qwen3 -> dense with q/k norms).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Any, BinaryIO, Dict, List, Optional, Tuple

import numpy as np
import torch

GGUF_MAGIC = 0x46554747          # "GGUF" little endian
QK = 32
QK_K = 256

# ggml type id -> (name, block elements, block bytes)
GGML_TYPES: Dict[int, Tuple[str, int, int]] = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22), 8: ("Q8_0", 32, 34),
    12: ("Q4_K", 256, 144), 13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210), 30: ("BF16", 1, 2),
}
_TYPE_ID = {v[0]: k for k, v in GGML_TYPES.items()}

# metadata value types
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


@dataclass
class GGUFTensorInfo:
    name: str
    shape: Tuple[int, ...]          # row-major (outermost first), i.e. reversed ggml ``ne``
    ggml_type: int
    offset: int                     # relative to the start of the data section


class GGUFFile:
    """Random access to the tensors and metadata of one GGUF file."""

    def __init__(self, path: str):
        self.path = path
        self.meta: Dict[str, Any] = {}
        self.tensors: Dict[str, GGUFTensorInfo] = {}
        with open(path, "rb") as f:
            magic, version = struct.unpack("<II", f.read(8))
            if magic != GGUF_MAGIC:
                raise ValueError(f"{path}: not a GGUF file")
            if version not in (2, 3):
                raise ValueError(f"{path}: unsupported GGUF version {version}")
            n_tensors, n_kv = struct.unpack("<QQ", f.read(16))
            for _ in range(n_kv):
                key = self._str(f)
                (vt,) = struct.unpack("<I", f.read(4))
                self.meta[key] = self._value(f, vt)
            for _ in range(n_tensors):
                name = self._str(f)
                (nd,) = struct.unpack("<I", f.read(4))
                ne = struct.unpack(f"<{nd}Q", f.read(8 * nd))
                t, off = struct.unpack("<IQ", f.read(12))
                self.tensors[name] = GGUFTensorInfo(name, tuple(reversed(ne)), t, off)
            align = int(self.meta.get("general.alignment", 32))
            pos = f.tell()
            self.data_start = (pos + align - 1) // align * align
        self._mm = np.memmap(path, dtype=np.uint8, mode="r")

    @staticmethod
    def _str(f: BinaryIO) -> str:
        (n,) = struct.unpack("<Q", f.read(8))
        return f.read(n).decode("utf-8", errors="replace")

    def _value(self, f: BinaryIO, vt: int):
        if vt in _SCALARS:
            fmt = _SCALARS[vt]
            return struct.unpack(fmt, f.read(struct.calcsize(fmt)))[0]
        if vt == 8:
            return self._str(f)
        if vt == 9:
            et, n = struct.unpack("<IQ", f.read(12))
            if et in _SCALARS:
                fmt = _SCALARS[et]
                sz = struct.calcsize(fmt)
                return list(struct.unpack(f"<{n}{fmt[1]}", f.read(sz * n)))
            return [self._value(f, et) for _ in range(n)]
        raise ValueError(f"GGUF metadata value type {vt}")

    def keys(self) -> List[str]:
        return list(self.tensors)

    def get(self, name: str, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        info = self.tensors[name]
        if info.ggml_type not in GGML_TYPES:
            raise ValueError(f"{name}: ggml type {info.ggml_type} is not supported")
        tname, bel, bby = GGML_TYPES[info.ggml_type]
        n = int(np.prod(info.shape)) if info.shape else 1
        nbytes = n // bel * bby
        raw = np.asarray(self._mm[self.data_start + info.offset:self.data_start + info.offset + nbytes])
        return dequantize(raw, tname, n).reshape(info.shape).to(dtype)


# ----------------------------------------------------------------------------- block formats
def _f16(a: np.ndarray) -> np.ndarray:
    return a.view(np.float16).astype(np.float32)


def _k_scale_min(sc: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """The 12-byte packed (scale, min) table of a Q4_K / Q5_K super-block -> two ``[nb, 8]`` uint8 arrays."""
    d = np.empty((sc.shape[0], 8), np.uint8)
    m = np.empty((sc.shape[0], 8), np.uint8)
    d[:, :4] = sc[:, 0:4] & 63
    m[:, :4] = sc[:, 4:8] & 63
    d[:, 4:] = (sc[:, 8:12] & 0x0F) | ((sc[:, 0:4] >> 6) << 4)
    m[:, 4:] = (sc[:, 8:12] >> 4) | ((sc[:, 4:8] >> 6) << 4)
    return d, m


def dequantize(raw: np.ndarray, tname: str, n: int) -> torch.Tensor:
    """``raw`` bytes of ``n`` elements in ggml format ``tname`` -> fp32 tensor ``[n]``."""
    if tname == "F32":
        return torch.from_numpy(raw.view(np.float32).copy())
    if tname == "F16":
        return torch.from_numpy(raw.view(np.float16).astype(np.float32))
    if tname == "BF16":
        return torch.from_numpy(raw.view(np.int16).copy()).view(torch.bfloat16).float()
    if tname == "Q8_0":
        b = raw.reshape(-1, 34)
        d = _f16(b[:, :2].copy()).reshape(-1, 1)
        return torch.from_numpy((b[:, 2:].view(np.int8).astype(np.float32) * d).reshape(-1))
    if tname in ("Q4_0", "Q4_1"):
        bs = 18 if tname == "Q4_0" else 20
        b = raw.reshape(-1, bs)
        d = _f16(b[:, :2].copy()).reshape(-1, 1)
        q = b[:, bs - 16:]
        lo, hi = (q & 0x0F).astype(np.float32), (q >> 4).astype(np.float32)
        x = np.concatenate([lo, hi], 1)
        if tname == "Q4_0":
            x = (x - 8.0) * d
        else:
            x = x * d + _f16(b[:, 2:4].copy()).reshape(-1, 1)
        return torch.from_numpy(x.reshape(-1))
    if tname == "Q5_0":
        b = raw.reshape(-1, 22)
        d = _f16(b[:, :2].copy()).reshape(-1, 1)
        qh = b[:, 2:6].copy().view(np.uint32).reshape(-1, 1)
        q = b[:, 6:]
        bit = ((qh >> np.arange(32, dtype=np.uint32)[None]) & 1).astype(np.uint8)
        lo = (q & 0x0F) | (bit[:, :16] << 4)
        hi = (q >> 4) | (bit[:, 16:] << 4)
        x = (np.concatenate([lo, hi], 1).astype(np.float32) - 16.0) * d
        return torch.from_numpy(x.reshape(-1))
    if tname in ("Q4_K", "Q5_K"):
        bs = 144 if tname == "Q4_K" else 176
        b = raw.reshape(-1, bs)
        d = _f16(b[:, 0:2].copy()).reshape(-1, 1)
        dmin = _f16(b[:, 2:4].copy()).reshape(-1, 1)
        sc, mn = _k_scale_min(b[:, 4:16])
        if tname == "Q4_K":
            qs = b[:, 16:144].reshape(-1, 4, 32)                     # 4 chunks of 64 values: low nibbles then high
            q = np.stack([qs & 0x0F, qs >> 4], 2).reshape(-1, 8, 32).astype(np.float32)
        else:
            qh = b[:, 16:48]                                          # one high bit per value, bit j of byte l -> sub-block j
            qs = b[:, 48:176].reshape(-1, 4, 32)
            lo, hi = qs & 0x0F, qs >> 4
            q = np.stack([lo, hi], 2).reshape(-1, 8, 32)
            hb = ((qh[:, None, :] >> np.arange(8, dtype=np.uint8)[None, :, None]) & 1).astype(np.uint8)
            q = (q | (hb << 4)).astype(np.float32)
        x = q * (d * sc.astype(np.float32))[:, :, None] - (dmin * mn.astype(np.float32))[:, :, None]
        return torch.from_numpy(x.reshape(-1))
    if tname == "Q6_K":
        b = raw.reshape(-1, 210)
        ql, qh = b[:, :128].reshape(-1, 2, 64), b[:, 128:192].reshape(-1, 2, 32)
        sc = b[:, 192:208].view(np.int8).astype(np.float32).reshape(-1, 2, 8)
        d = _f16(b[:, 208:210].copy()).reshape(-1, 1, 1)
        l0, l1 = ql[:, :, :32], ql[:, :, 32:]
        q1 = (l0 & 0x0F) | ((qh & 3) << 4)
        q2 = (l1 & 0x0F) | (((qh >> 2) & 3) << 4)
        q3 = (l0 >> 4) | (((qh >> 4) & 3) << 4)
        q4 = (l1 >> 4) | (((qh >> 6) & 3) << 4)
        q = np.stack([q1, q2, q3, q4], 2).astype(np.float32) - 32.0   # [nb, 2, 4, 32]: 128-value halves of four 32-value runs
        s = sc.reshape(-1, 2, 4, 2)                                    # scale index = run * 2 + (position // 16)
        s = np.repeat(s, 16, axis=3)                                   # [nb, 2, 4, 32]
        return torch.from_numpy((q * s * d[..., None]).reshape(-1))
    raise ValueError(f"ggml type {tname} is not supported")


# ----------------------------------------------------------------------------- writers (tests, export)
def quantize_q8_0(x: torch.Tensor) -> np.ndarray:
    v = x.float().reshape(-1, QK).numpy()
    d = np.abs(v).max(1, keepdims=True) / 127.0
    q = np.where(d > 0, np.round(v / np.where(d > 0, d, 1.0)), 0).astype(np.int8)
    out = np.empty((v.shape[0], 34), np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def quantize_q4_0(x: torch.Tensor) -> np.ndarray:
    v = x.float().reshape(-1, QK).numpy()
    idx = np.abs(v).argmax(1)
    mx = v[np.arange(v.shape[0]), idx]
    d = (mx / -8.0).astype(np.float16).astype(np.float32)
    inv = np.where(d != 0, 1.0 / np.where(d != 0, d, 1.0), 0.0)
    q = np.clip(np.floor(v * inv[:, None] + 8.5), 0, 15).astype(np.uint8)
    out = np.empty((v.shape[0], 18), np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


def write_gguf(path: str, meta: Dict[str, Any], tensors: Dict[str, Tuple[torch.Tensor, str]], alignment: int = 32) -> None:
    """Minimal GGUF v3 writer: ``tensors[name] = (tensor, type)`` with type in F32 / F16 / BF16 / Q8_0 / Q4_0."""
    def s(b: str) -> bytes:
        e = b.encode()
        return struct.pack("<Q", len(e)) + e

    def val(v) -> bytes:
        if isinstance(v, bool):
            return struct.pack("<I?", 7, v)
        if isinstance(v, int):
            return struct.pack("<Iq", 11, v) if v < 0 else struct.pack("<II", 4, v)
        if isinstance(v, float):
            return struct.pack("<If", 6, v)
        if isinstance(v, str):
            return struct.pack("<I", 8) + s(v)
        if isinstance(v, (list, tuple)):
            if all(isinstance(e, int) for e in v):
                return struct.pack("<IIQ", 9, 5, len(v)) + struct.pack(f"<{len(v)}i", *v)
            if all(isinstance(e, str) for e in v):
                return struct.pack("<IIQ", 9, 8, len(v)) + b"".join(s(e) for e in v)
        raise TypeError(type(v))
    blobs, infos, off = [], [], 0
    for name, (t, tname) in tensors.items():
        if tname == "F32":
            raw = t.float().contiguous().numpy().tobytes()
        elif tname == "F16":
            raw = t.half().contiguous().numpy().tobytes()
        elif tname == "BF16":
            raw = t.bfloat16().contiguous().view(torch.int16).numpy().tobytes()
        elif tname == "Q8_0":
            raw = quantize_q8_0(t).tobytes()
        elif tname == "Q4_0":
            raw = quantize_q4_0(t).tobytes()
        else:
            raise ValueError(tname)
        ne = tuple(reversed(t.shape))
        infos.append(s(name) + struct.pack("<I", len(ne)) + struct.pack(f"<{len(ne)}Q", *ne) + struct.pack("<IQ", _TYPE_ID[tname], off))
        pad = (-len(raw)) % alignment
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    meta = dict(meta)
    meta.setdefault("general.alignment", alignment)
    head = struct.pack("<IIQQ", GGUF_MAGIC, 3, len(tensors), len(meta))
    head += b"".join(s(k) + val(v) for k, v in meta.items()) + b"".join(infos)
    head += b"\0" * ((-len(head)) % alignment)
    with open(path, "wb") as f:
        f.write(head)
        for b in blobs:
            f.write(b)


# ----------------------------------------------------------------------------- model mapping
_ARCH_TO_TYPE = {"llama": "llama", "mistral": "mistral", "qwen2": "qwen2", "qwen3": "qwen3"}


def config_from_gguf(g: GGUFFile):
    """``ModelConfig`` from the file's ``<arch>.*`` metadata."""
    from ..config import ModelConfig
    arch = str(g.meta.get("general.architecture", "llama"))
    if arch not in _ARCH_TO_TYPE:
        raise ValueError(f"GGUF architecture '{arch}' is not supported (known: {sorted(_ARCH_TO_TYPE)})")
    m = lambda k, d=None: g.meta.get(f"{arch}.{k}", d)
    nh = int(m("attention.head_count"))
    hs = int(m("embedding_length"))
    vocab = int(m("vocab_size", 0)) or len(g.meta.get("tokenizer.ggml.tokens", [])) or g.tensors["token_embd.weight"].shape[0]
    hd = int(m("attention.key_length", hs // nh))
    return ModelConfig(model_type=_ARCH_TO_TYPE[arch], family="dense", vocab_size=vocab, hidden_size=hs,
                       intermediate_size=int(m("feed_forward_length")), num_hidden_layers=int(m("block_count")),
                       num_attention_heads=nh, num_key_value_heads=int(m("attention.head_count_kv", nh)), head_dim=hd,
                       rms_norm_eps=float(m("attention.layer_norm_rms_epsilon", 1e-5)), rope_theta=float(m("rope.freq_base", 10000.0)),
                       max_position_embeddings=int(m("context_length", 4096)), qk_norm=arch == "qwen3",
                       attention_bias=arch == "qwen2", tie_word_embeddings="output.weight" not in g.tensors,
                       bos_token_id=g.meta.get("tokenizer.ggml.bos_token_id"), eos_token_id=g.meta.get("tokenizer.ggml.eos_token_id"))


def _unpermute_rope_rows(w: torch.Tensor, n_head: int) -> torch.Tensor:
    """Inverse of the llama GGUF converter's q/k row permutation (interleaved rotary pairs -> half-split layout)."""
    rows = w.shape[0]
    d = rows // n_head
    return w.reshape(n_head, d // 2, 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


def load_gguf_model(path: str, pctx=None, device="cpu", dtype: Optional[str] = None, max_pos: Optional[int] = None,
                    quant: Optional[str] = None):
    """Build a decoder from a GGUF file.  ``quant`` ("fp8_block" / "nvfp4") re-quantises the de-quantised projection
    weights for the engine's tensor-core GEMMs; default keeps them in the model dtype."""
    from ..config import QuantConfig
    from ..models import build_model
    g = GGUFFile(path)
    cfg = config_from_gguf(g)
    if dtype:
        cfg.dtype = dtype
    if quant:
        cfg.quant = QuantConfig(method=quant)
    model = build_model(cfg, pctx, device=device, with_mtp=False)
    dt = model.dtype
    arch = str(g.meta.get("general.architecture", "llama"))
    permuted = arch in ("llama", "mistral")
    get = lambda n: g.get(n, torch.float32)
    has = lambda n: n in g.tensors
    model.embed = get("token_embd.weight").to(device=model.device, dtype=dt)
    for i, layer in enumerate(model.layers):
        p = f"blk.{i}"
        q, k = get(f"{p}.attn_q.weight"), get(f"{p}.attn_k.weight")
        if permuted:
            q, k = _unpermute_rope_rows(q, cfg.num_attention_heads), _unpermute_rope_rows(k, cfg.num_key_value_heads)
        bias = None
        if has(f"{p}.attn_q.bias"):
            bq, bk, bv = get(f"{p}.attn_q.bias"), get(f"{p}.attn_k.bias"), get(f"{p}.attn_v.bias")
            if permuted:
                bq, bk = _unpermute_rope_rows(bq, cfg.num_attention_heads), _unpermute_rope_rows(bk, cfg.num_key_value_heads)
            r, tp, mx = layer.mixer.pctx.tp_rank, layer.mixer.pctx.tp_size, layer.mixer
            kv0 = ((r // mx.kv_rep) * mx.hkv) * mx.d if tp > 1 else 0
            bias = torch.cat([bq[r * mx.hq * mx.d:(r + 1) * mx.hq * mx.d], bk[kv0:kv0 + mx.hkv * mx.d],
                              bv[kv0:kv0 + mx.hkv * mx.d]]).to(device=model.device, dtype=dt)
        to = lambda t: t.to(device=model.device, dtype=dt)
        qn = to(get(f"{p}.attn_q_norm.weight")) if has(f"{p}.attn_q_norm.weight") else None
        kn = to(get(f"{p}.attn_k_norm.weight")) if has(f"{p}.attn_k_norm.weight") else None
        layer.mixer.load(to(q), to(k), to(get(f"{p}.attn_v.weight")), to(get(f"{p}.attn_output.weight")), qn, kn, bias)
        layer.ffn.load(to(get(f"{p}.ffn_gate.weight")), to(get(f"{p}.ffn_up.weight")), to(get(f"{p}.ffn_down.weight")))
        layer.input_norm = to(get(f"{p}.attn_norm.weight"))
        layer.post_norm = to(get(f"{p}.ffn_norm.weight"))
    model.final_norm = get("output_norm.weight").to(device=model.device, dtype=dt)
    head = get("output.weight") if has("output.weight") else model.embed
    model.set_lm_head(head.to(device=model.device, dtype=dt))
    model.mtp = None
    model.finalize(max_pos)
    return model
