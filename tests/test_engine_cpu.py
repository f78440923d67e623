"""CPU plumbing: tiny random-init decoders through the paged, continuously-batched engine must
reproduce a plain eager forward (greedy tokens and logits)."""
import pytest
import torch

from atlas_b200.config import EngineConfig, tiny_deepseek, tiny_dense, tiny_hybrid, tiny_moe, tiny_nemotron_h
from atlas_b200.engine import LLMEngine
from atlas_b200.models import ForwardBatch, build_model
from atlas_b200.sampling import SamplingParams


def _prompts(n=4, length=32, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 1024, (length,), generator=g).tolist() for _ in range(n)]


def _eager_greedy(model, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(model.forward_dense_reference(toks)[-1].argmax()))
    return toks[len(prompt):]


@pytest.mark.parametrize("mk", [tiny_dense, tiny_moe, tiny_hybrid, tiny_nemotron_h, tiny_deepseek])
def test_engine_matches_eager_greedy(mk):
    model = build_model(mk()).init_random(0)
    eng = LLMEngine(model, EngineConfig(block_size=16, num_kv_blocks=64, max_num_seqs=8, max_prefill_tokens=48))
    prompts = _prompts()
    outs = eng.generate(prompts, SamplingParams(max_tokens=16, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.output_tokens == _eager_greedy(model, p, 16)
        assert o.finish_reason == "length"
    eng.pool.check_invariants()


@pytest.mark.parametrize("mk", [tiny_dense, tiny_moe, tiny_hybrid, tiny_nemotron_h, tiny_deepseek])
def test_paged_chunked_logits_match_eager(mk):
    model = build_model(mk()).init_random(0)
    toks = _prompts(1, 40)[0]
    full = model.forward_dense_reference(toks)
    cache = model.alloc_cache(8, 16, torch.float32, state_slots=2)
    bt = [[5, 2, 7]]
    fb = ForwardBatch.build([toks[:25]], [0], bt, 16, state_slots=[1], has_state=[False], all_logits=True)
    l1 = model.compute_logits(model.forward(fb, cache))
    fb = ForwardBatch.build([toks[25:]], [25], bt, 16, state_slots=[1], has_state=[True], all_logits=True)
    l2 = model.compute_logits(model.forward(fb, cache))
    torch.testing.assert_close(torch.cat([l1, l2]), full, atol=2e-5, rtol=1e-4)


def test_speculative_equals_plain_greedy():
    model = build_model(tiny_hybrid()).init_random(0)
    prompts = _prompts()
    base = LLMEngine(model, EngineConfig(num_kv_blocks=64, max_num_seqs=8)).generate(
        prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    spec = LLMEngine(model, EngineConfig(num_kv_blocks=64, max_num_seqs=8, speculative=True, num_drafts=3,
                                         mtp_gate=False))
    outs = spec.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    assert [o.output_tokens for o in outs] == [o.output_tokens for o in base]
    assert spec.stats.spec_proposed > 0


def test_dcut_prunes_verify_rows_and_stays_lossless():
    """Verify-depth planning from drafter confidence: fewer rows are verified, the output is still plain greedy."""
    model = build_model(tiny_hybrid()).init_random(0)
    prompts = _prompts()
    sp = SamplingParams(max_tokens=12, ignore_eos=True)
    base = LLMEngine(model, EngineConfig(num_kv_blocks=64, max_num_seqs=8)).generate(prompts, sp)
    full = LLMEngine(model, EngineConfig(num_kv_blocks=64, max_num_seqs=8, speculative=True, num_drafts=3, mtp_gate=False))
    full.generate(prompts, sp)
    cut = LLMEngine(model, EngineConfig(num_kv_blocks=64, max_num_seqs=8, speculative=True, num_drafts=3, mtp_gate=False,
                                        dcut_ratio=0.5))
    outs = cut.generate(prompts, sp)
    assert [o.output_tokens for o in outs] == [o.output_tokens for o in base]
    assert cut.spec.dcut_pruned > 0 and 0 < cut.stats.spec_proposed < full.stats.spec_proposed


def test_order_independence_with_sampling():
    """A seeded request draws the same tokens whatever else shares its batch."""
    model = build_model(tiny_dense()).init_random(0)
    prompts = _prompts(6)
    sp = [SamplingParams(max_tokens=10, temperature=0.8, top_p=0.9, top_k=50, seed=100 + i, ignore_eos=True)
          for i in range(6)]
    e1 = LLMEngine(model, EngineConfig(num_kv_blocks=128, max_num_seqs=8))
    all_out = e1.generate(prompts, samplings=sp)
    for i in (0, 3, 5):
        e = LLMEngine(model, EngineConfig(num_kv_blocks=128, max_num_seqs=8))
        solo = e.generate([prompts[i]], samplings=[sp[i]])[0]
        assert solo.output_tokens == all_out[i].output_tokens


@pytest.mark.parametrize("mk", [tiny_dense, tiny_hybrid, tiny_nemotron_h])
def test_ngram_speculation_equals_plain_greedy(mk):
    """Prompt-lookup drafts never change the output (acceptance compares against the target's own samples) and are
    actually accepted on repetitive text."""
    model = build_model(mk()).init_random(0)
    g = torch.Generator().manual_seed(9)
    base_piece = torch.randint(0, 1024, (12,), generator=g).tolist()
    prompts = [base_piece * 4, torch.randint(0, 1024, (40,), generator=g).tolist(), (base_piece[:5] * 9)[:44]]
    # a bias towards three token ids makes the (random-init) model repeat itself, so lookups hit
    sp = SamplingParams(max_tokens=24, ignore_eos=True, logit_bias={5: 40.0, 6: 40.0, 7: 40.0})
    want = [o.output_tokens for o in LLMEngine(model, EngineConfig(num_kv_blocks=96, max_num_seqs=8)).generate(prompts, sp)]
    eng = LLMEngine(model, EngineConfig(num_kv_blocks=96, max_num_seqs=8, ngram_speculative=True, num_drafts=3, mtp_gate=False))
    got = [o.output_tokens for o in eng.generate(prompts, sp)]
    assert got == want
    assert eng.stats.spec_proposed > 0 and eng.stats.spec_accepted > 0
    eng.pool.check_invariants()


@pytest.mark.parametrize("keep", [1.0, 0.5])
def test_self_speculation_equals_plain_greedy(keep):
    """Layer-skipping drafts from the target itself: the output is always plain greedy (the target verifies every draft);
    with no layer skipped the drafter IS the target, so nearly every draft is accepted, which checks the draft pass's
    positions, KV writes and chaining; with half the layers the machinery still runs and stays lossless."""
    from atlas_b200.sched.spec import SelfSpecController, skip_layer_ids
    assert skip_layer_ids(32, 0.5)[0] == 0 and skip_layer_ids(32, 0.5)[-1] == 31 and len(skip_layer_ids(32, 0.5)) == 16
    assert skip_layer_ids(4, 1.0) == [0, 1, 2, 3] and skip_layer_ids(5, 0.1) == [0, 4]
    model = build_model(tiny_dense()).init_random(0)
    prompts = _prompts()
    sp = SamplingParams(max_tokens=16, ignore_eos=True)
    base = LLMEngine(model, EngineConfig(num_kv_blocks=96, max_num_seqs=8)).generate(prompts, sp)
    eng = LLMEngine(model, EngineConfig(num_kv_blocks=96, max_num_seqs=8, self_speculative=True, self_spec_keep=keep,
                                        num_drafts=3, mtp_gate=False))
    assert isinstance(eng.spec, SelfSpecController)
    outs = eng.generate(prompts, sp)
    assert [o.output_tokens for o in outs] == [o.output_tokens for o in base]
    assert eng.stats.spec_proposed > 0
    if keep == 1.0:
        assert eng.stats.spec_accepted >= 0.9 * eng.stats.spec_proposed, (eng.stats.spec_accepted, eng.stats.spec_proposed)
    eng.pool.check_invariants()
    # recurrent layers would be advanced by a draft pass: such models do not get this proposer
    hyb = build_model(tiny_hybrid()).init_random(0)
    assert not SelfSpecController.supported(hyb)
    assert LLMEngine(hyb, EngineConfig(num_kv_blocks=64, max_num_seqs=8, self_speculative=True, num_drafts=3)).spec is None


def test_ngram_proposer_lookup():
    from atlas_b200.sched.sequence import Sequence
    from atlas_b200.sched.spec import NgramSpecController

    class _E:      # the proposer only needs the configuration
        pass
    ctl = NgramSpecController(_E(), EngineConfig(ngram_speculative=True, num_drafts=3, ngram_max=3, ngram_min=2))
    seq = Sequence("r", [1, 2, 3, 4, 5, 9, 9, 2, 3, 4], SamplingParams(max_tokens=32))
    assert ctl.propose(seq) == [5, 9, 9]            # "2 3 4" was followed by 5 9 9
    seq.output_tokens += [5, 9]
    assert ctl.propose(seq) == [9, 2, 3]            # "4 5 9" -> after its earlier occurrence come 9 2 3
    seq.output_tokens += [7]
    assert ctl.propose(seq) == []                   # nothing ends in "9 7"


def test_rotated_kv_cache_keeps_attention_and_spends_fp8_range_better():
    """The "turbo8" cache: heads rotated by the orthonormal Walsh-Hadamard transform before the cache write.  With a
    full-precision cache the attention output (rotated back) equals the plain one; with an FP8 cache and an outlier
    channel in the keys the rotated cache is the more accurate of the two."""
    from atlas_b200 import ops
    from atlas_b200.models.batch import ForwardBatch
    from atlas_b200.ops import reference as ref
    torch.manual_seed(0)
    T, Hq, Hkv, D, bs = 40, 4, 2, 64, 16
    h = ref.hadamard(D)
    assert torch.allclose(h @ h, torch.eye(D), atol=1e-6)                 # orthonormal and its own inverse
    q, k, v = torch.randn(T, Hq, D), torch.randn(T, Hkv, D), torch.randn(T, Hkv, D)
    k[:, :, 7] *= 30.0                                                    # an outlier channel
    q[:, :, 7] *= 0.05
    rope = ref.build_rope_cache(D, 64, 1e4, None, "cpu")
    fb = ForwardBatch.build([[0] * T], [0], [[0, 1, 2]], bs)

    def run(dtype, rotate, k_scale=1.0):
        kc, vc = torch.zeros(4, bs, Hkv, D, dtype=dtype), torch.zeros(4, bs, Hkv, D, dtype=dtype)
        qr = ops.qk_norm_rope_kv_write(q.clone(), k, v, fb.positions.int(), rope, D, kc, vc, fb.slot_mapping.int(), k_scale, 1.0,
                                       rotate=rotate)
        out = ops.paged_attention(qr, kc, vc, fb, D ** -0.5, k_scale, 1.0)
        return ops.head_rotate(out) if rotate else out
    exact = run(torch.float32, False)
    assert torch.allclose(run(torch.float32, True), exact, atol=2e-4)
    err_plain = (run(torch.float8_e4m3fn, False, 0.25) - exact).pow(2).mean().sqrt()
    err_rot = (run(torch.float8_e4m3fn, True, 0.25) - exact).pow(2).mean().sqrt()
    assert err_rot < err_plain


def test_engine_with_rotated_fp8_cache():
    cfg = tiny_dense()
    eng = LLMEngine(build_model(cfg).init_random(0), EngineConfig(num_kv_blocks=64, max_num_seqs=4, kv_cache_dtype="turbo8"))
    assert eng.kv_dtype == torch.float8_e4m3fn and all(l.mixer.kv_rotate for l in eng.model.layers)
    plain = LLMEngine(build_model(cfg).init_random(0), EngineConfig(num_kv_blocks=64, max_num_seqs=4, kv_cache_dtype="fp8"))
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 1024, (24,), generator=g).tolist() for _ in range(3)]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    a = [o.output_tokens for o in eng.generate(prompts, sp)]
    b = [o.output_tokens for o in plain.generate(prompts, sp)]
    assert all(len(x) == 6 for x in a)
    assert sum(x[0] == y[0] for x, y in zip(a, b)) >= 2        # same model, two roundings of the same cache contents


def test_reduced_vocabulary_draft_head_is_lossless_and_ranked_rows_cover_more(tmp_path):
    """A draft head over a subset of the vocabulary changes which drafts are proposed, never what is emitted; rows ranked
    by a recorded frequency table (forced ids kept) accept more than the first rows by id."""
    from atlas_b200.utils.vocab_rank import VocabRecorder, coverage, load_ranked_ids, select_rows
    model = build_model(tiny_hybrid()).init_random(0)
    prompts = _prompts()
    sp = SamplingParams(max_tokens=12, ignore_eos=True)
    base = LLMEngine(model, EngineConfig(num_kv_blocks=64, max_num_seqs=8)).generate(prompts, sp)
    want = [o.output_tokens for o in base]
    rec = VocabRecorder()
    for o in base:
        rec.add(o.output_tokens)
    table = str(tmp_path / "rank.json")
    rec.save(table)
    ranked = load_ranked_ids(table)
    assert ranked[0] == rec.counts.most_common(1)[0][0] or rec.counts[ranked[0]] == rec.counts.most_common(1)[0][1]
    rows = select_rows(64, 1024, ranked, forced=(1023,))
    assert rows == sorted(rows) and len(rows) == 64 and 1023 in rows
    emitted = [t for o in want for t in o]
    assert coverage(rows, emitted) > coverage(select_rows(64, 1024), emitted)

    def run(**kw):
        eng = LLMEngine(build_model(tiny_hybrid()).init_random(0),
                        EngineConfig(num_kv_blocks=64, max_num_seqs=8, speculative=True, num_drafts=3, mtp_gate=False, **kw))
        outs = eng.generate(prompts, sp)
        assert [o.output_tokens for o in outs] == want
        return eng
    full = run()
    whole = run(mtp_draft_vocab=1023)                       # nearly the whole vocabulary: drafts as good as the full head's
    by_id = run(mtp_draft_vocab=64)
    by_freq = run(mtp_draft_vocab=64, mtp_vocab_rank=table)
    assert by_id.model.draft_rows == 64 and by_freq.model.draft_rows == 64 and getattr(full.model, "draft_head", None) is None
    assert whole.stats.spec_accepted >= full.stats.spec_accepted - 2
    assert by_freq.stats.spec_accepted >= by_id.stats.spec_accepted
    cut = run(mtp_draft_vocab=64, mtp_vocab_rank=table, dcut_ratio=0.5)       # confidence taken over the reduced rows
    assert cut.spec.dcut_pruned > 0
