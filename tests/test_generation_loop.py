"""The generation loop's decisions, on the CPU: how requests are cut into batches,
when sequences stop, what the callback sees, what goes back to the cache."""
import pytest

import gpt_fast_b200 as gf
from gpt_fast_b200.engine.generate import _plan_batches, cache_tokens_needed
import plain_llama


@pytest.fixture
def tiny(plain_kernels, tiny_folders):
    model = gf.load(tiny_folders["tiny-a"], dtype="float32", device="cpu")
    p, cfg = plain_llama.load_folder(tiny_folders["tiny-a"])
    return model, p, cfg


def test_batches_are_cut_in_order():
    assert _plan_batches(7, 3) == [[0, 1, 2], [3, 4, 5], [6]]
    assert _plan_batches(2, 5) == [[0, 1]]
    with pytest.raises(ValueError):
        _plan_batches(3, 0)
    # the largest batch sizes the cache: whole pages per sequence
    assert cache_tokens_needed([5, 70, 64, 1], 10, 2, 64) == 64 + 128
    assert cache_tokens_needed([5, 70, 64, 1], 10, 4, 64) == 64 + 128 + 128 + 64


def test_token_budget_and_order(tiny):
    model, p, cfg = tiny
    prompts = [[3, 4, 5], [9], [7, 7, 7, 7, 7, 7]]
    seqs, stats = gf.generate(model, prompts, 5, temperature=0.0, stop_tokens=[])
    for pr, s in zip(prompts, seqs):
        assert s[:len(pr)] == pr and len(s) == len(pr) + 5                       # exactly N new tokens
        assert s[len(pr):] == plain_llama.greedy_generate(pr, 5, p, cfg)
    assert stats.batches == 1 and stats.decode_steps == 4 and stats.decode_tokens == 12
    assert stats.prompt_tokens == 10 and stats.generated_tokens == 15


def test_a_stop_token_ends_only_its_sequence_and_the_batch_goes_on(tiny):
    model, p, cfg = tiny
    prompts = [[3, 4, 5], [9, 1], [100, 101, 102, 103]]
    free, _ = gf.generate(model, prompts, 8, temperature=0.0, stop_tokens=[])
    stop = free[1][2 + 2]                                                         # request 1's third new token
    seen = []
    seqs, stats = gf.generate(model, prompts, 8, temperature=0.0, stop_tokens=[stop],
                              callback=lambda ids, toks: seen.append((list(ids), toks.tolist())))
    for pr, f, s in zip(prompts, free, seqs):
        new = f[len(pr):]
        cut = new.index(stop) + 1 if stop in new else len(new)
        assert s == pr + new[:cut]
    assert len(seqs[1]) == 2 + 3
    assert seen[0][0] == [0, 1, 2]                                                # after the prefill: everyone
    gone = next(i for i, (ids, _) in enumerate(seen) if 1 not in ids)
    assert all(1 not in ids for ids, _ in seen[gone:])                           # once out, never back
    assert sum(len(ids) for ids, _ in seen) == stats.generated_tokens


def test_a_stop_token_from_the_prefill_ends_the_sequence_at_once(tiny):
    model, p, cfg = tiny
    prompts = [[3, 4, 5], [9, 1]]
    free, _ = gf.generate(model, prompts, 4, temperature=0.0, stop_tokens=[])
    seqs, stats = gf.generate(model, prompts, 4, temperature=0.0, stop_tokens=[free[0][3]])
    assert seqs[0] == prompts[0] + [free[0][3]]
    if free[0][3] not in free[1][2:]:
        assert seqs[1] == free[1]


def test_batches_follow_one_another_on_one_cache(tiny):
    model, p, cfg = tiny
    prompts = [[i + 1, i + 2] for i in range(5)]
    cache = model.new_cache(max_tokens=64 * 2, max_seqs=2)
    seqs, stats = gf.generate(model, prompts, 3, temperature=0.0, batch_size=2, cache=cache, stop_tokens=[])
    assert stats.batches == 3
    assert cache.slots.n_free == cache.n_slots and cache.pages_free == cache.n_pages
    alone = [gf.generate(model, [pr], 3, temperature=0.0, stop_tokens=[])[0][0] for pr in prompts]
    assert seqs == alone
    from gpt_fast_b200.cache import CacheFull
    with pytest.raises(CacheFull):
        gf.generate(model, prompts, 3, temperature=0.0, batch_size=3, cache=cache)
    assert cache.slots.n_free == cache.n_slots and cache.pages_free == cache.n_pages   # given back after the error


def test_default_stop_tokens_come_from_the_config(plain_kernels, tmp_path):
    cfg = gf.config_from_name("tiny-a")
    free_dir = gf.write_model_folder(str(tmp_path / "free"), cfg, seed=11)
    free_model = gf.load(free_dir, dtype="float32", device="cpu")
    free, _ = gf.generate(free_model, [[3, 4, 5]], 6, temperature=0.0)
    cfg["eos_token_id"] = free[0][3 + 1]
    stop_dir = gf.write_model_folder(str(tmp_path / "stop"), cfg, seed=11)
    model = gf.load(stop_dir, dtype="float32", device="cpu")
    assert model.spec.stop_tokens == (free[0][4],)
    seqs, _ = gf.generate(model, [[3, 4, 5]], 6, temperature=0.0)
    new = free[0][3:]
    assert seqs[0] == [3, 4, 5] + new[:new.index(free[0][4]) + 1]
    seqs, _ = gf.generate(model, [[3, 4, 5]], 6, temperature=0.0, stop_tokens=[])
    assert seqs[0] == free[0]


def test_bad_requests_are_refused(tiny):
    model, _, _ = tiny
    with pytest.raises(ValueError, match="at least one token"):
        gf.generate(model, [[1], []], 3)
    with pytest.raises(ValueError, match="max_new_tokens"):
        gf.generate(model, [[1]], 0)
    assert gf.generate(model, [], 3)[0] == []
    st = gf.Stepper(model, model.new_cache(max_tokens=128))
    slots = st.cache.begin(2)
    with pytest.raises(ValueError, match="twice"):
        st.step([slots[0], slots[0]], [[1], [2]])
    with pytest.raises(ValueError, match="place 3"):
        st.step(slots, [[1, 2], [3]], want=[[3], []])
    with pytest.raises(ValueError, match="at least one token"):
        st.step(slots, [[1], []])
    st.step(slots, [[1, 300], [2]])                                             # id 300 is outside tiny-a's vocabulary
    with pytest.raises(gf.ops.KernelError, match="token id out of range"):
        st.check()


def test_decode_slice_count_follows_its_cost_model():
    """How many slices a decode step cuts a sequence's cache into (a host-side decision, no GPU needed)."""
    from gpt_fast_b200.ops.cuda import decode_slices
    sms = 148
    assert decode_slices(130, 64, 64, sms) == 1                      # three pages: nothing to cut
    assert decode_slices(4001, 64, 64, sms) == 4                     # 64 blocks x 4 = one round of 256 blocks
    assert decode_slices(32001, 64, 8, sms) == 37                    # one sequence: as many blocks as fit in one round
    assert decode_slices(2001, 64, 512, sms) == 1                    # the grid is large already
    for ctx in (1, 63, 64, 65, 1000, 5000, 100000):
        for blocks in (1, 8, 64, 512, 4096):
            s = decode_slices(ctx, 64, blocks, sms)
            pages = -(-ctx // 64)
            assert 1 <= s <= 48 and (s == 1 or pages // s >= 4)      # a slice keeps at least four pages
