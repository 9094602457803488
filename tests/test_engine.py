"""Host-side logic of the continuous-batching engine: the page pool (C ABI), the sampler, the repetition
check and the slot loop with a stand-in model.  No GPU, no kernels."""
import random

import pytest
import torch
from hypothesis import given, settings, strategies as st

from kinetics_b200.engine import (Engine, PagePool, PoolExhausted, recent_subseq_repeat_check,
                                  sample_next_tokens)

PAGE = 16


# ---------------------------------------------------------------- page pool against a Python model

class ModelPool:
    def __init__(self, num_pages, max_slots):
        self.free = list(range(num_pages - 1, -1, -1))
        self.pages = {s: None for s in range(max_slots)}
        self.tokens = {s: -1 for s in range(max_slots)}
        self.reserved = {s: 0 for s in range(max_slots)}

    def promised(self):
        return sum(self.reserved[s] - len(self.pages[s]) for s in self.pages if self.tokens[s] >= 0)

    def unpromised(self):
        return len(self.free) - self.promised()


def _need(t):
    return (t + PAGE - 1) // PAGE


@settings(max_examples=60, deadline=None)
@given(st.integers(4, 40), st.integers(1, 6), st.lists(st.tuples(st.integers(0, 3), st.integers(0, 5),
                                                                 st.integers(0, 200), st.integers(0, 80)),
                                                       min_size=1, max_size=60))
def test_pool_matches_a_python_model(num_pages, max_slots, script):
    pool, model = PagePool(num_pages, max_slots), ModelPool(num_pages, max_slots)
    for op, slot, a, b in script:
        slot %= max_slots
        if op == 0:                                       # admit
            now, most = a % 100, a % 100 + b
            ok = model.tokens[slot] < 0 and _need(most) <= model.unpromised()
            if model.tokens[slot] >= 0:
                with pytest.raises(Exception):
                    pool.admit(slot, now, most)
                continue
            if not ok:
                with pytest.raises(PoolExhausted):
                    pool.admit(slot, now, most)
                continue
            pool.admit(slot, now, most)
            model.pages[slot] = [model.free.pop() for _ in range(_need(now))]
            model.tokens[slot], model.reserved[slot] = now, _need(most)
        elif op == 1:                                     # extend one slot
            d = b % 20
            if model.tokens[slot] < 0:
                with pytest.raises(Exception):
                    pool.extend([slot], d)
                continue
            if _need(model.tokens[slot] + d) > model.reserved[slot]:
                with pytest.raises(PoolExhausted):
                    pool.extend([slot], d)
                continue
            pool.extend([slot], d)                        # inside the promise: never fails
            model.tokens[slot] += d
            while len(model.pages[slot]) < _need(model.tokens[slot]):
                model.pages[slot].append(model.free.pop())
        elif op == 2:                                     # release
            if model.tokens[slot] < 0:
                with pytest.raises(Exception):
                    pool.release(slot)
                continue
            pool.release(slot)
            model.free.extend(reversed(model.pages[slot]))
            model.pages[slot], model.tokens[slot], model.reserved[slot] = None, -1, 0
        else:                                             # export every live slot, in a shuffled order
            live = [s for s in range(max_slots) if model.tokens[s] >= 0]
            random.Random(a).shuffle(live)
            idx, indptr, last = pool.export(live)
            want = [p for s in live for p in model.pages[s]]
            assert idx.tolist() == want
            assert indptr.tolist() == [0] + [sum(len(model.pages[s]) for s in live[:i + 1]) for i in range(len(live))]
            assert last.tolist() == [0 if model.tokens[s] == 0 else (model.tokens[s] - 1) % PAGE + 1 for s in live]
        # invariants after every operation
        held = [p for s in model.pages if model.tokens[s] >= 0 for p in model.pages[s]]
        assert len(held) == len(set(held)) and not set(held) & set(model.free)
        assert len(held) + len(model.free) == num_pages
        assert pool.free_pages == model.unpromised() >= 0
        for s in range(max_slots):
            assert pool.tokens(s) == model.tokens[s]
    pool.close()


def test_pool_rejects_bad_arguments():
    with pytest.raises(ValueError):
        PagePool(0, 4)
    pool = PagePool(8, 2)
    with pytest.raises(Exception):
        pool.admit(5, 1, 1)
    with pytest.raises(Exception):
        pool.admit(0, 10, 5)                     # more now than ever
    pool.admit(0, 16, 32)
    with pytest.raises(PoolExhausted):
        pool.extend([0], 17)                     # beyond the promise
    assert pool.tokens(0) == 16                  # nothing changed
    pool.extend([0], 16)
    assert pool.pages(0) == 2 and pool.free_pages == 6


# ---------------------------------------------------------------- sampler, repetition check

def test_sampler_greedy_and_degenerate_cases():
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(5, 1, 50, generator=g)
    arg = logits.argmax(-1)
    assert torch.equal(sample_next_tokens(logits, 0.0, 0, 1.0), arg)
    assert torch.equal(sample_next_tokens(logits, 0.7, 1, 1.0, g), arg)          # top-k = 1
    assert torch.equal(sample_next_tokens(logits, 0.7, 0, 1e-6, g), arg)         # the nucleus is one token


def test_sampler_respects_topk_and_nucleus():
    g = torch.Generator().manual_seed(1)
    logits = torch.randn(64, 1, 100, generator=g) * 3
    out = sample_next_tokens(logits, 1.0, 5, 1.0, g)
    top5 = logits.squeeze(1).topk(5, -1).indices
    assert (out == top5).any(-1).all()
    # nucleus 0.5 at temperature 1: the drawn token lies in the shortest prefix whose mass reaches 0.5
    out = sample_next_tokens(logits, 1.0, 0, 0.5, g)
    probs = torch.softmax(logits.squeeze(1), -1)
    sp, si = probs.sort(-1, descending=True)
    keep = (sp.cumsum(-1) - sp) < 0.5                     # tokens that start before the mass is reached
    for b in range(64):
        assert int(out[b]) in si[b][keep[b]].tolist()


def test_sampler_distribution():
    g = torch.Generator().manual_seed(2)
    logits = torch.log(torch.tensor([0.6, 0.3, 0.1])).reshape(1, 1, 3).repeat(20000, 1, 1)
    out = sample_next_tokens(logits, 1.0, 0, 1.0, g).reshape(-1)
    freq = torch.bincount(out, minlength=3).float() / out.numel()
    assert torch.allclose(freq, torch.tensor([0.6, 0.3, 0.1]), atol=0.02)


@settings(max_examples=80, deadline=None)
@given(st.lists(st.integers(0, 2), min_size=0, max_size=60), st.integers(1, 5), st.integers(1, 30), st.integers(1, 4))
def test_repeat_check_matches_brute_force(tokens, sub, window, thresh):
    t = torch.tensor(tokens, dtype=torch.long)
    n = len(tokens)
    want = False
    if n >= sub:
        w = tokens[max(0, n - window - sub): n - sub]
        if len(w) >= sub:
            recent = tokens[n - sub:]
            want = sum(w[i:i + sub] == recent for i in range(len(w) - sub + 1)) >= thresh
    assert recent_subseq_repeat_check(t, sub, window, thresh) == want


# ---------------------------------------------------------------- the slot loop with a stand-in model

VOCAB, EOS = 64, 63


class CountingModel:
    """next token = (last token + 1) mod VOCAB, whatever the history: outputs are known in advance."""

    def __init__(self):
        self.calls = []

    def inference(self, input_ids, position_ids, batch_idx, kv):
        self.calls.append((tuple(batch_idx.tolist()), input_ids.shape[1]))
        kv.saw(batch_idx.tolist(), input_ids.shape[1])
        nxt = (input_ids + 1) % VOCAB
        return torch.nn.functional.one_hot(nxt, VOCAB).float() * 10.0


class HostKV:
    """Keeps only what the engine needs from a KV manager; admission through a real PagePool."""

    def __init__(self, max_batch_size, num_pages):
        self.max_batch_size = max_batch_size
        self.pool = PagePool(num_pages, max_batch_size)
        self.lengths = [0] * max_batch_size
        self.peak_active = 0

    def can_admit(self, total):
        return self.pool.can_admit(total)

    def admit(self, slot, prompt_len, total):
        self.pool.admit(slot, 0, total)

    def begin_step(self, slots):
        self.peak_active = max(self.peak_active, len(slots))

    def saw(self, slots, n):
        self.pool.extend(slots, n)
        for s in slots:
            self.lengths[s] += n

    def clear_cache(self, slot):
        self.lengths[slot] = 0
        if self.pool.tokens(slot) >= 0:
            self.pool.release(slot)


def _expected(prompt, max_new):
    out, t, n = [], prompt[-1], 1
    while True:                 # the engine stops on the step whose sampled token is EOS or at max_new tokens
        t = (t + 1) % VOCAB
        out.append(t)
        nxt = (t + 1) % VOCAB
        n += 1
        if nxt == EOS or n >= max_new:
            return out


@pytest.mark.parametrize("num_pages,slots", [(64, 4), (6, 4), (3, 2)])
def test_engine_loop_serves_every_request(num_pages, slots):
    rng = random.Random(3)
    requests = [{"id": i, "input_ids": [rng.randrange(0, 60) for _ in range(rng.randrange(1, 20))]} for i in range(11)]
    max_new = 12
    kv, model = HostKV(slots, num_pages), CountingModel()
    eng = Engine(model, kv, max_seq_len=64, device="cpu", temperature=0.0, eos=[EOS], repeat_check=False)
    done = eng.offline_exec(requests, max_new)
    assert sorted(r["id"] for r in done) == list(range(11))
    for r in done:
        assert r["output_tokens"] == _expected(r["input_ids"], max_new), r
    # every page is back, every slot is free, and the pool bounded how many sequences ran together
    assert kv.pool.free_pages == num_pages and not any(eng.slots_occupy_status)
    assert kv.peak_active <= slots
    if num_pages == 3:          # 19 + 12 tokens need 2 pages: never more than one such sequence at a time
        assert kv.peak_active <= 2
    # prefills are single-sequence calls, decodes one token for all active slots
    assert all(n == 1 or len(s) == 1 for s, n in model.calls)


def test_preprocess_hook_sees_every_request_once_even_when_it_waits_for_pages():
    # a hook that is not idempotent (it prepends a token): a request that waits for pages must not be
    # preprocessed again on every refill attempt
    rng = random.Random(5)
    requests = [{"id": i, "input_ids": [rng.randrange(1, 60) for _ in range(rng.randrange(10, 20))]} for i in range(7)]
    seen = []

    def prepend(req):
        seen.append(req["id"])
        req["input_ids"] = [0] + list(req["input_ids"])

    kv, model = HostKV(4, 3), CountingModel()           # 3 pages: requests queue up behind one another
    eng = Engine(model, kv, max_seq_len=64, device="cpu", temperature=0.0, eos=[EOS], repeat_check=False,
                 preprocess=prepend)
    done = eng.offline_exec(requests, 12)
    assert sorted(seen) == list(range(7))
    assert all(r["input_ids"][0] == 0 and r["input_ids"][1] != 0 for r in done)


def test_engine_refuses_a_request_that_can_never_fit():
    kv, model = HostKV(2, 1), CountingModel()
    eng = Engine(model, kv, max_seq_len=64, device="cpu", eos=[EOS], repeat_check=False)
    with pytest.raises(PoolExhausted):
        eng.offline_exec([{"input_ids": list(range(20))}], 12)


def test_engine_stops_a_repeating_sequence():
    class Stuck:
        def inference(self, input_ids, position_ids, batch_idx, kv):
            return torch.nn.functional.one_hot(torch.full_like(input_ids, 7), VOCAB).float()

    class NoKV:
        max_batch_size = 1

        def clear_cache(self, slot):
            pass

    eng = Engine(Stuck(), NoKV(), max_seq_len=256, device="cpu", eos=[EOS], repeat_check=True,
                 repeat_check_window=32, repeat_block_size=8)
    done = eng.offline_exec([{"input_ids": [1, 2, 3]}], 200)
    # the check starts once more than 32 tokens exist and trims the last block of 8
    assert len(done) == 1 and 20 < len(done[0]["output_tokens"]) < 60
    assert set(done[0]["output_tokens"]) == {7}


def test_merge_of_the_ranks_vocabulary_maxima_is_the_global_argmax():
    """Greedy sampling over a vocabulary projection split by rows over the ranks: the merge of the ranks'
    (maximum, token id) pairs equals the argmax over the whole row, ties going to the lowest id."""
    import torch
    from kinetics_b200.decoder_stack import merge_rank_maxima
    g = torch.Generator().manual_seed(3)
    ranks, rows, vocab = 4, 64, 1024
    logits = torch.randint(-5, 6, (rows, vocab), generator=g).float()          # many exact ties
    per = vocab // ranks
    pairs = []
    for r in range(ranks):
        vals, idx = logits[:, r * per:(r + 1) * per].max(dim=-1)
        first = (logits[:, r * per:(r + 1) * per] == vals[:, None]).float().argmax(dim=-1)   # lowest id of the maximum
        pairs.append(torch.stack((vals, (first + r * per).float()), dim=1))
    got = merge_rank_maxima(torch.stack(pairs))
    want = (logits == logits.max(dim=-1, keepdim=True).values).float().argmax(dim=-1)
    assert torch.equal(got, want)
