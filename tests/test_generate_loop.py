"""The generation loop's decisions, with a scripted backend instead of a device."""
import pytest

from janus_b200.engine.generate import plan_batch, run_generation, tokens_held
from janus_b200.sampling import SamplerConfig


class ScriptedBackend:
    """Next token of request r after k generated tokens is script[r][k]."""

    def __init__(self, script, n_slots):
        self.script, self.free = script, list(range(n_slots))
        self.held, self.log, self.max_live = {}, [], 0

    def alloc_slot(self):
        s = self.free.pop()
        assert s not in self.held
        self.held[s] = 0
        self.max_live = max(self.max_live, len(self.held))
        return s

    def free_slot(self, s):
        assert s in self.held, "slot freed twice"
        del self.held[s]
        self.free.append(s)

    def synchronize(self):
        pass

    def prefill(self, slots, prompts, requests):
        self.log.append(("prefill", list(requests), [len(p) for p in prompts]))
        for s, p in zip(slots, prompts):
            assert self.held[s] == 0
            self.held[s] = len(p)
        return [self.script[r][0] for r in requests]

    def decode(self, slots, last, requests, steps):
        self.log.append(("decode", list(requests), list(steps)))
        for s, r, t, k in zip(slots, requests, last, steps):
            assert t == self.script[r][k - 1]            # the token fed is the one just produced
            self.held[s] += 1
        return [self.script[r][k] for r, k in zip(requests, steps)]


def run(script, prompts, max_new, stop=(), batch=8, cap=10_000, max_seq=1000, slots=8, cb=None):
    b = ScriptedBackend(script, slots)
    out = run_generation(b, prompts, max_new, stop, batch, cap, max_seq, slots, 64, cb)
    assert not b.held, "a slot was never given back"
    return b, out


def test_unequal_prompts_stop_tokens_and_early_finish():
    script = {0: [5, 6, 99, 1], 1: [99, 1, 1, 1], 2: [7, 8, 9, 10]}
    b, (toks, reasons, stats) = run(script, [[1] * 3, [1] * 10, [1] * 5], 4, stop=[99])
    assert toks == [[5, 6], [], [7, 8, 9, 10]]            # the stop token is not part of the output
    assert reasons == ["stop", "stop", "length"]
    assert b.log[0] == ("prefill", [0, 1, 2], [3, 10, 5])
    assert [e[1] for e in b.log[1:]] == [[0, 2], [0, 2], [2]]   # finished sequences leave the batch
    assert stats.decode_steps == 3 and stats.decode_tokens == 5 and stats.prefill_tokens == 18
    assert stats.batches == 1


def test_batches_follow_one_another():
    script = {r: [r + 1] * 10 for r in range(5)}
    b, (toks, reasons, stats) = run(script, [[1, 2]] * 5, 3, batch=2)
    assert stats.batches == 3 and b.max_live == 2
    assert toks == [[r + 1] * 3 for r in range(5)] and reasons == ["length"] * 5
    assert [e[1] for e in b.log if e[0] == "prefill"] == [[0, 1], [2, 3], [4]]


def test_capacity_limits_the_batch_and_errors_when_nothing_fits():
    # each request holds 64 * ceil((60 + 9) / 64) = 128 tokens
    assert tokens_held(60, 10, 64) == 128
    assert plan_batch([0, 1, 2], [60, 60, 60], 10, 8, 256, 8, 64) == [0, 1]
    assert plan_batch([0, 1, 2], [60, 60, 60], 10, 8, 10_000, 1, 64) == [0]
    with pytest.raises(ValueError, match="request 0"):
        plan_batch([0], [60], 10, 8, 64, 8, 64)


def test_budgets():
    script = {0: list(range(10, 30))}
    _, (toks, reasons, _) = run(script, [[1, 2, 3]], 0)
    assert toks == [[]]
    _, (toks, reasons, _) = run(script, [[1, 2, 3]], 1)
    assert toks == [[10]] and reasons == ["length"]
    # the longest sequence ends generation: 3 prompt tokens, room for 5 positions
    b, (toks, reasons, _) = run(script, [[1, 2, 3]], 20, max_seq=5)
    assert toks == [[10, 11, 12]] and reasons == ["length"]
    assert max(b.log[-1][2]) == 2                          # the last token produced is never fed
    with pytest.raises(ValueError, match="empty"):
        run(script, [[]], 3)
    with pytest.raises(ValueError, match="longest"):
        run(script, [[1] * 9], 3, max_seq=5)


def test_callback_can_end_a_request():
    script = {0: [1, 2, 3, 4], 1: [5, 6, 7, 8]}
    seen = []

    def cb(r, t):
        seen.append((r, t))
        return not (r == 0 and t == 2)

    _, (toks, reasons, _) = run(script, [[9], [9]], 4, cb=cb)
    assert toks == [[1, 2], [5, 6, 7, 8]] and reasons == ["stop", "length"]
    assert (0, 3) not in seen


class RunAheadBackend(ScriptedBackend):
    """A backend that can launch a step before the one before was read; a token
    -1 stands for what the step before produced for that slot."""

    def __init__(self, script, n_slots):
        super().__init__(script, n_slots)
        self.last = {}          # slot -> token produced last ("on the device")
        self.in_flight = 0
        self.max_in_flight = 0
        self.wasted_rows = 0

    def prefill(self, slots, prompts, requests):
        out = super().prefill(slots, prompts, requests)
        self.last.update(dict(zip(slots, out)))
        return out

    def decode_launch(self, slots, tokens, requests, steps):
        fed = [self.last[s] if t == -1 else t for s, t in zip(slots, tokens)]
        for s in slots:
            assert s in self.held, "a step was launched for a slot that was given back"
        out = self.decode(slots, fed, requests, steps)
        self.last.update(dict(zip(slots, out)))
        self.in_flight += 1
        self.max_in_flight = max(self.max_in_flight, self.in_flight)
        return out

    def decode_collect(self, handle):
        self.in_flight -= 1
        return handle


@pytest.mark.parametrize("case", range(4))
def test_run_ahead_loop_gives_the_plain_loop_s_results(case):
    import random
    rng = random.Random(case)
    n = 6
    script = {r: [rng.choice([1, 2, 3, 4, 99]) for _ in range(12)] for r in range(n)}
    prompts = [[7] * rng.randint(1, 9) for _ in range(n)]
    kw = dict(stop=[99], batch=3, max_seq=15, slots=4)
    _, plain = run(script, prompts, 8, **kw)
    b = RunAheadBackend(script, 4)
    ahead = run_generation(b, prompts, 8, [99], 3, 10_000, 15, 4, 64, None)
    assert not b.held and ahead[0] == plain[0] and ahead[1] == plain[1]
    assert ahead[2].decode_tokens == plain[2].decode_tokens and ahead[2].decode_steps == plain[2].decode_steps
    assert b.max_in_flight == 2                      # a step is launched while the one before is unread
    assert b.in_flight == 0


def test_sampler_config_names_and_checks():
    c = SamplerConfig()
    assert (c.temperature, c.top_k, c.top_p, c.beam_width, c.max_tokens) == (0.0, 0, 1.0, 1, 128)
    for bad in (dict(temperature=-1.0), dict(top_k=-1), dict(top_p=0.0), dict(top_p=1.5),
                dict(repetition_penalty=0.0), dict(beam_width=4), dict(max_tokens=-1)):
        with pytest.raises(ValueError):
            SamplerConfig(**bad).validate()


def _expected(script, prompt_len, max_new, stop, max_seq):
    """What a request must produce: its scripted tokens up to a stop token (not part of the output), its
    budget, or the longest sequence, whichever comes first."""
    out = []
    for tok in script:
        if tok in stop:
            return out, "stop"
        out.append(tok)
        if len(out) >= max_new or prompt_len + len(out) > max_seq:
            return out, "length"
    raise AssertionError("script too short")


def test_any_mix_of_requests_is_served_whole_and_every_slot_comes_back():
    """Property (hypothesis): whatever the prompts, budgets, stop tokens, batch size, slots and cache capacity,
    both loops give every request exactly its scripted tokens and reason, never hold more sequences than the
    batch size and the slots allow, never more tokens than the cache has, and give every slot back once."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=150, deadline=None)
    @given(st.data())
    def check(data):
        n = data.draw(st.integers(1, 9))
        max_new = data.draw(st.integers(1, 12))
        max_seq = data.draw(st.integers(16, 40))
        prompts = [[7] * data.draw(st.integers(1, 15)) for _ in range(n)]
        script = {r: [data.draw(st.sampled_from([1, 2, 3, 4, 5, 99])) for _ in range(max_new + 1)] for r in range(n)}
        slots = data.draw(st.integers(1, 5))
        batch = data.draw(st.integers(1, 6))
        page = 8
        biggest = max(tokens_held(len(p), max_new, page) for p in prompts)
        cap = data.draw(st.integers(biggest, 4 * biggest))
        want = [_expected(script[r], len(prompts[r]), max_new, {99}, max_seq) for r in range(n)]
        for backend_type in (ScriptedBackend, RunAheadBackend):
            b = backend_type(script, slots)
            toks, reasons, stats = run_generation(b, prompts, max_new, [99], batch, cap, max_seq, slots, page, None)
            assert toks == [w[0] for w in want] and reasons == [w[1] for w in want]
            assert not b.held and sorted(b.free) == list(range(slots))
            assert b.max_live <= min(batch, slots)
            for kind, reqs, _ in b.log:
                if kind == "prefill":          # what a batch may come to hold fits the cache
                    assert sum(tokens_held(len(prompts[r]), max_new, page) for r in reqs) <= cap
            assert stats.requests == n and stats.prefill_tokens == sum(len(p) for p in prompts)
    check()


@pytest.mark.parametrize("fail_in", ["callback", "decode", "prefill"])
def test_every_slot_comes_back_when_a_batch_ends_in_an_error(fail_in):
    """A callback that raises, or a step that raises in the middle of a batch, ends the call; no slot
    stays held, so the next call finds the whole cache again."""
    script = {r: [r + 1] * 10 for r in range(4)}

    class Failing(ScriptedBackend):
        def decode(self, slots, last, requests, steps):
            if fail_in == "decode" and max(steps) >= 2:
                raise RuntimeError("the step failed")
            return super().decode(slots, last, requests, steps)

        def prefill(self, slots, prompts, requests):
            if fail_in == "prefill":
                raise RuntimeError("the step failed")
            return super().prefill(slots, prompts, requests)

    def cb(request, token):
        if fail_in == "callback" and request == 1:
            raise KeyError("the caller's own fault")
        return True

    b = Failing(script, 4)
    with pytest.raises((RuntimeError, KeyError)):
        run_generation(b, [[1, 2]] * 4, 5, [], 4, 10_000, 1000, 4, 64, cb)
    assert not b.held and sorted(b.free) == [0, 1, 2, 3]
    # and the same backend serves the next call
    ok = ScriptedBackend(script, 4)
    ok.free, ok.held = b.free, b.held
    toks, reasons, stats = run_generation(ok, [[1, 2]] * 4, 3, [], 4, 10_000, 1000, 4, 64, None)
    assert toks == [[r + 1] * 3 for r in range(4)] and not ok.held


def test_prompt_steps_hold_every_token_once_in_order_within_the_limit():
    """`plan_prompt_steps`: each prompt's pieces are consecutive, in order and complete; no step exceeds the
    limit; every step but the last is full; without a limit (or under it) there is one step of whole prompts."""
    import random

    from janus_b200.engine.generate import plan_prompt_steps
    assert plan_prompt_steps([5, 3], None) == [[(0, 0, 5), (1, 0, 3)]]
    assert plan_prompt_steps([5, 3], 8) == [[(0, 0, 5), (1, 0, 3)]]
    assert plan_prompt_steps([5, 3], 4) == [[(0, 0, 4)], [(0, 4, 5), (1, 0, 3)]]
    assert plan_prompt_steps([2, 9, 1], 3) == [[(0, 0, 2), (1, 0, 1)], [(1, 1, 4)], [(1, 4, 7)], [(1, 7, 9), (2, 0, 1)]]
    rng = random.Random(4)
    for _ in range(200):
        lens = [rng.randint(1, 50) for _ in range(rng.randint(1, 8))]
        limit = rng.randint(1, 60)
        steps = plan_prompt_steps(lens, limit)
        sizes = [sum(b - a for _, a, b in st) for st in steps]
        assert all(0 < n <= limit for n in sizes) and (sum(lens) <= limit or all(n == limit for n in sizes[:-1]))
        pieces = [piece for st in steps for piece in st]
        assert [i for i, _, _ in pieces] == sorted(i for i, _, _ in pieces)
        for i, n in enumerate(lens):
            mine = [(a, b) for j, a, b in pieces if j == i]
            assert mine[0][0] == 0 and mine[-1][1] == n and all(x[1] == y[0] for x, y in zip(mine, mine[1:]))
            assert all(b > a for a, b in mine)
            where = [k for k, st in enumerate(steps) for j, _, _ in st if j == i]
            assert where == list(range(where[0], where[0] + len(where)))
