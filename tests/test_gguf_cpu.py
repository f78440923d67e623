"""GGUF container: block de-quantisers against their definitions, and a tiny model written to a GGUF file (llama
row permutation included) that must reproduce the logits of the same weights loaded directly."""
import numpy as np
import pytest
import torch

from atlas_b200.config import ModelConfig
from atlas_b200.loader import gguf as G
from atlas_b200.models import build_model


def test_block_formats_roundtrip():
    torch.manual_seed(0)
    x = torch.randn(8, 256)
    for tname, tol in (("Q8_0", 6e-3), ("Q4_0", 1.2e-1)):
        raw = (G.quantize_q8_0 if tname == "Q8_0" else G.quantize_q4_0)(x)
        y = G.dequantize(np.frombuffer(raw.tobytes(), dtype=np.uint8), tname, x.numel()).reshape(x.shape)
        assert float((y - x).norm() / x.norm()) < tol, tname
    # F16 / BF16 / F32 are exact up to their own rounding
    for tname, ref in (("F32", x), ("F16", x.half().float()), ("BF16", x.bfloat16().float())):
        raw = {"F32": x.numpy().tobytes(), "F16": x.half().numpy().tobytes(),
               "BF16": x.bfloat16().view(torch.int16).numpy().tobytes()}[tname]
        y = G.dequantize(np.frombuffer(raw, dtype=np.uint8), tname, x.numel()).reshape(x.shape)
        assert torch.equal(y, ref)


def _pack_q4_k(d, dmin, sc, mn, q):
    """Super-blocks from their parts (scales / mins 6-bit, quants 4-bit), in the layout the reader expects."""
    nb = d.shape[0]
    out = np.zeros((nb, 144), np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(nb, 2)
    out[:, 2:4] = dmin.astype(np.float16).view(np.uint8).reshape(nb, 2)
    s = out[:, 4:16]
    s[:, 0:4] = (sc[:, :4] & 63) | ((sc[:, 4:] >> 4) << 6)
    s[:, 4:8] = (mn[:, :4] & 63) | ((mn[:, 4:] >> 4) << 6)
    s[:, 8:12] = (sc[:, 4:] & 0x0F) | ((mn[:, 4:] & 0x0F) << 4)
    qq = q.reshape(nb, 4, 2, 32)
    out[:, 16:144] = (qq[:, :, 0] | (qq[:, :, 1] << 4)).reshape(nb, 128)
    return out


def test_k_quant_decoders_match_their_definition():
    rng = np.random.default_rng(1)
    nb = 5
    d = rng.uniform(0.01, 0.1, nb).astype(np.float16).astype(np.float32)
    dmin = rng.uniform(0.01, 0.1, nb).astype(np.float16).astype(np.float32)
    sc = rng.integers(0, 64, (nb, 8)).astype(np.uint8)
    mn = rng.integers(0, 64, (nb, 8)).astype(np.uint8)
    q = rng.integers(0, 16, (nb, 8, 32)).astype(np.uint8)
    want = q.astype(np.float32) * (d[:, None] * sc)[:, :, None] - (dmin[:, None] * mn)[:, :, None]
    got = G.dequantize(_pack_q4_k(d, dmin, sc, mn, q).reshape(-1), "Q4_K", nb * 256).numpy().reshape(nb, 8, 32)
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)
    # Q6_K: value index i of a 256-block -> half = i // 128, run = (i % 128) // 32, pos = i % 32
    ql = rng.integers(0, 256, (nb, 128)).astype(np.uint8)
    qh = rng.integers(0, 256, (nb, 64)).astype(np.uint8)
    s6 = rng.integers(-32, 32, (nb, 16)).astype(np.int8)
    d6 = rng.uniform(0.01, 0.1, nb).astype(np.float16)
    blk = np.concatenate([ql, qh, s6.view(np.uint8), d6.view(np.uint8).reshape(nb, 2)], 1)
    got6 = G.dequantize(blk.reshape(-1), "Q6_K", nb * 256).numpy().reshape(nb, 256)
    want6 = np.zeros((nb, 256), np.float32)
    for b in range(nb):
        for half in range(2):
            for l in range(32):
                lo0, lo1 = ql[b, half * 64 + l], ql[b, half * 64 + 32 + l]
                h = qh[b, half * 32 + l]
                vals = [(lo0 & 0xF) | ((h & 3) << 4), (lo1 & 0xF) | (((h >> 2) & 3) << 4), (lo0 >> 4) | (((h >> 4) & 3) << 4),
                        (lo1 >> 4) | (((h >> 6) & 3) << 4)]
                for run, v in enumerate(vals):
                    scale = s6[b, half * 8 + run * 2 + l // 16]
                    want6[b, half * 128 + run * 32 + l] = float(d6[b]) * scale * (int(v) - 32)
    np.testing.assert_allclose(got6, want6, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("arch,wtype", [("llama", "F32"), ("qwen3", "F16"), ("llama", "Q8_0")])
def test_model_from_gguf_matches_direct_load(arch, wtype, tmp_path):
    cfg = ModelConfig(model_type=arch, family="dense", vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64, rope_theta=1e4, rms_norm_eps=1e-5,
                      max_position_embeddings=256, qk_norm=arch == "qwen3", dtype="float32")
    ref = build_model(cfg).init_random(3)
    H, d = cfg.hidden_size, cfg.head_dim

    def permute(w, n_head):          # what the llama converter does to q / k rows
        return w.reshape(n_head, 2, w.shape[0] // n_head // 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)
    tensors = {"token_embd.weight": (ref.embed, "F32"), "output_norm.weight": (ref.final_norm, "F32"),
               "output.weight": (ref.lm_head.weight, wtype)}
    deq = {}

    def put(name, w, kind=wtype):
        tensors[name] = (w.contiguous(), kind)
    for i, l in enumerate(ref.layers):
        nq, nkv = cfg.num_attention_heads * d, cfg.num_key_value_heads * d
        qkv = l.mixer.qkv.weight
        q, k, v = qkv[:nq], qkv[nq:nq + nkv], qkv[nq + nkv:nq + 2 * nkv]
        if arch == "llama":
            q, k = permute(q, cfg.num_attention_heads), permute(k, cfg.num_key_value_heads)
        put(f"blk.{i}.attn_q.weight", q); put(f"blk.{i}.attn_k.weight", k); put(f"blk.{i}.attn_v.weight", v)
        put(f"blk.{i}.attn_output.weight", l.mixer.o.weight)
        I = cfg.intermediate_size
        put(f"blk.{i}.ffn_gate.weight", l.ffn.gate_up.weight[:I]); put(f"blk.{i}.ffn_up.weight", l.ffn.gate_up.weight[I:])
        put(f"blk.{i}.ffn_down.weight", l.ffn.down.weight)
        put(f"blk.{i}.attn_norm.weight", l.input_norm, "F32"); put(f"blk.{i}.ffn_norm.weight", l.post_norm, "F32")
        if arch == "qwen3":
            put(f"blk.{i}.attn_q_norm.weight", l.mixer.q_norm, "F32"); put(f"blk.{i}.attn_k_norm.weight", l.mixer.k_norm, "F32")
    meta = {"general.architecture": arch, f"{arch}.block_count": 2, f"{arch}.embedding_length": H,
            f"{arch}.feed_forward_length": cfg.intermediate_size, f"{arch}.attention.head_count": 4,
            f"{arch}.attention.head_count_kv": 2, f"{arch}.attention.key_length": d, f"{arch}.attention.layer_norm_rms_epsilon": 1e-5,
            f"{arch}.rope.freq_base": 1e4, f"{arch}.context_length": 256, f"{arch}.vocab_size": 512}
    path = str(tmp_path / "m.gguf")
    G.write_gguf(path, meta, tensors)
    got = G.load_gguf_model(path, dtype="float32")
    toks = torch.randint(0, 512, (20,), generator=torch.Generator().manual_seed(1)).tolist()
    a, b = ref.forward_dense_reference(toks), got.forward_dense_reference(toks)
    if wtype == "F32":
        torch.testing.assert_close(b, a, atol=1e-5, rtol=1e-5)
    else:
        rel = float((a - b).norm() / a.norm())
        assert rel < (2e-3 if wtype == "F16" else 3e-2), rel
        assert (a.argmax(-1) == b.argmax(-1)).float().mean() > 0.9
