"""Block-selected decode attention: summaries from the cache, forced + scored selection, exactness inside the budget,
and the engine option."""
import math

import torch

from atlas_b200.config import EngineConfig, tiny_dense
from atlas_b200.engine import LLMEngine
from atlas_b200.kv.sparse_select import BlockSelector, attend_selected
from atlas_b200.models import build_model
from atlas_b200.models.batch import ForwardBatch
from atlas_b200.ops import reference as ref
from atlas_b200.sampling import SamplingParams


def _attn(q, kc, vc, fb, scale, ks, vs, window):
    return ref.paged_attention(q, kc, vc, fb.block_tables, fb.seq_lens, fb.query_start_loc, scale, ks, vs, window)


def test_selection_keeps_the_blocks_that_carry_the_attention_mass():
    torch.manual_seed(0)
    bs, hkv, hq, d, nb = 16, 2, 4, 32, 40
    L = 20 * bs + 5                                     # 21 blocks, the last one partial
    table = torch.randperm(nb)[:21].tolist()
    kc = torch.randn(nb, bs, hkv, d) * 0.1
    vc = torch.randn(nb, bs, hkv, d)
    q = torch.randn(1, hq, d)
    hot = [7, 13]                                       # two middle blocks whose keys line up with the query
    for j in hot:
        kc[table[j]] += q.view(hkv, hq // hkv, d).mean(1)[None] * 3.0
    fb = ForwardBatch.build([[0]], [L - 1], [table], bs)
    sel = BlockSelector(nb, bs, budget_blocks=6, sink=1, recent=2)
    fbp = ForwardBatch.build([[0] * L], [0], [table], bs)         # "prefill" wrote every block: summarise them
    sel.on_write(0, kc, fbp)
    assert float(sel.count[0][table[20]]) == 5 and float(sel.count[0][table[3]]) == bs
    torch.testing.assert_close(sel.key_sum[0][table[3]], kc[table[3]].sum(0))
    tab, lens = sel.select(0, q, fb.block_tables, fb.seq_lens)
    picked = tab[0].tolist()
    assert picked[0] == table[0] and picked[-2:] == [table[19], table[20]]          # sink, recent (partial block last)
    assert table[7] in picked and table[13] in picked and int(lens[0]) == 5 * bs + 5
    full = _attn(q, kc, vc, fb, 1 / math.sqrt(d), 1.0, 1.0, None)
    sparse = attend_selected(_attn, sel, 0, q, kc, vc, fb, 1 / math.sqrt(d), 1.0, 1.0, None)
    # almost all softmax mass sits in the hot blocks, so 6 of 21 blocks reproduce the output closely
    assert float((full - sparse).norm() / full.norm()) < 0.05
    # within the budget nothing changes at all
    wide = BlockSelector(nb, bs, budget_blocks=32)
    wide.on_write(0, kc, fbp)
    same = attend_selected(_attn, wide, 0, q, kc, vc, fb, 1 / math.sqrt(d), 1.0, 1.0, None)
    torch.testing.assert_close(same, full, atol=0, rtol=0)


def test_engine_option_is_exact_within_budget_and_bounded_beyond():
    model = build_model(tiny_dense("float32"), device="cpu").init_random(0)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, model.cfg.vocab_size, (n,), generator=g).tolist() for n in (70, 33)]
    sp = SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True)
    base_cfg = dict(num_kv_blocks=64, max_num_seqs=4, max_seq_len=128, enable_prefix_caching=False)
    dense = LLMEngine(model, EngineConfig(**base_cfg)).generate(prompts, sp)
    wide = LLMEngine(model, EngineConfig(sparse_attention_blocks=16, **base_cfg))
    out = wide.generate(prompts, sp)
    assert [o.output_tokens for o in out] == [o.output_tokens for o in dense]       # 5 blocks < budget: identical
    narrow = LLMEngine(model, EngineConfig(sparse_attention_blocks=4, **base_cfg))
    out2 = narrow.generate(prompts, sp)
    assert all(len(o.output_tokens) == 10 for o in out2) and narrow.selector.selected_steps > 0
    for l in model.layers:
        l.mixer.selector = None
