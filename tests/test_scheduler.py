"""The scheduler's decisions, from traces of integers: budget, portions,
promotion, deferral, what happens when pages run out, cancels, the latency
guard, and record/replay."""
import numpy as np
import pytest

from alofa_b200.engine.scheduler import Action, SchedConfig, SchedInput, Scheduler, format_config, format_tick, parse_config, replay_trace
from alofa_b200.errors import AlofaError


class Pool:
    """A stand-in for the cache manager's book of one group of pages: what the
    engine would do with every action (reserve, free, give back)."""

    def __init__(self, sched, page=16, capacity=8):
        self.sched, self.page, self.capacity = sched, page, capacity
        self.len = {}

    def free(self):
        return [self.capacity - sum(-(-n // self.page) for n in self.len.values())]

    def apply(self, act: Action):
        for rid in act.preempted:
            self.len.pop(rid, None)
        for rid in act.decode:
            self.len[rid] += 1
        for rid, start, end in act.prefill:
            assert self.len.get(rid, 0) == start, "portions must be contiguous"
            self.len[rid] = end
        assert self.free()[0] >= 0, "the action over-committed the pool"
        for rid in act.finished:
            self.len.pop(rid, None)


def run(cfg, arrivals_by_tick, ticks, capacity=None, cancels_by_tick=None):
    sched = Scheduler(cfg)
    pool = Pool(sched, cfg.groups[0][0], cfg.groups[0][2])
    lines, acts, waiting = [format_config(cfg)], [], []
    for t in range(ticks):
        waiting += arrivals_by_tick.get(t, [])
        cancels = (cancels_by_tick or {}).get(t, [])
        for rid in cancels:
            pool.len.pop(rid, None)
        inp = SchedInput(list(waiting), cancels, [], pool.free())
        act = sched.step(inp)
        waiting = [a for a, st in zip(waiting, act.arrival_status) if st == 0]
        pool.apply(act)
        assert act.tokens() <= cfg.token_budget
        lines.append(format_tick(inp, act))
        acts.append(act)
    return sched, acts, "\n".join(lines)


def test_long_prompt_is_cut_into_portions_and_first_token_comes_with_the_last():
    cfg = SchedConfig(token_budget=32, max_chunk=16, max_batch=4, max_tokens=128, watermark_permille=1000, groups=[(16, 0, 8)])
    sched, acts, _ = run(cfg, {0: [(1, 40, 3)]}, 8)
    assert acts[0].prefill == [(1, 0, 16)] and acts[1].prefill == [(1, 16, 32)] and acts[2].prefill == [(1, 32, 40)]
    assert acts[3].decode == [1] and acts[4].decode == [1] and acts[4].finished == [1]  # 1 + 2 decoded = 3 tokens
    assert acts[5].tokens() == 0 and sched.counts()["live"] == 0


def test_max_new_of_one_finishes_with_its_prompt():
    cfg = SchedConfig(token_budget=64, max_chunk=64, max_batch=2, max_tokens=128, groups=[(16, 0, 8)])
    _, acts, _ = run(cfg, {0: [(5, 9, 1)]}, 3)
    assert acts[0].prefill == [(5, 0, 9)] and acts[0].finished == [5] and acts[1].tokens() == 0


def test_decode_goes_before_prefill_and_budget_is_shared():
    cfg = SchedConfig(token_budget=10, max_chunk=8, max_batch=4, max_tokens=128, groups=[(16, 0, 32)])
    _, acts, _ = run(cfg, {0: [(1, 4, 20), (2, 4, 20)], 2: [(3, 30, 5)]}, 6)
    assert acts[2].decode == [1, 2] and acts[2].prefill == [(3, 0, 8)]
    assert acts[3].decode == [1, 2] and acts[3].prefill == [(3, 8, 16)]
    for act in acts:
        assert act.tokens() <= 10


def test_committed_admission_defers_instead_of_refusing_and_never_preempts():
    cfg = SchedConfig(token_budget=64, max_chunk=32, max_batch=4, max_tokens=128, watermark_permille=1000, admission="committed", groups=[(16, 0, 8)])
    # each request may grow to 64 tokens = 4 pages: two fit beside each other
    sched, acts, _ = run(cfg, {0: [(1, 30, 34), (2, 30, 34), (3, 30, 34)]}, 90)
    assert acts[0].arrival_status == [1, 1, 0]
    assert all(not a.preempted for a in acts)
    done = [rid for a in acts for rid in a.finished]
    assert sorted(done) == [1, 2, 3] and done.index(3) == 2
    with pytest.raises(AlofaError) as err:
        sched.can_ever_fit(100, 100)
    assert err.value.code in ("capacity", "out_of_range")


def test_pages_run_out_newest_running_request_is_recomputed():
    cfg = SchedConfig(token_budget=64, max_chunk=32, max_batch=4, max_tokens=128, watermark_permille=1000, admission="optimistic", groups=[(16, 0, 6)])
    # three prompts of 30 (2 pages each) fill the pool; growth past 32 needs a third page each
    sched, acts, trace = run(cfg, {0: [(1, 30, 20), (2, 30, 20), (3, 30, 20)]}, 120)
    preempted = [rid for a in acts for rid in a.preempted]
    assert preempted and preempted[0] == 3, "the newest running request goes first"
    assert acts[-1].preempt_total == len(preempted)
    done = [rid for a in acts for rid in a.finished]
    assert sorted(done) == [1, 2, 3], "a preempted request is prefilled again and finishes"
    assert replay_trace(trace) == []


def test_a_lone_request_that_cannot_grow_fails_loudly():
    cfg = SchedConfig(token_budget=64, max_chunk=64, max_batch=2, max_tokens=128, admission="optimistic", groups=[(16, 0, 4)])
    sched = Scheduler(cfg)
    with pytest.raises(AlofaError, match="even alone"):
        sched.can_ever_fit(60, 10)
    act = sched.step(SchedInput([(1, 60, 10)], [], [], [4]))
    assert act.arrival_status[0] < 0


def test_watermark_preempts_down_to_the_limit():
    cfg = SchedConfig(token_budget=64, max_chunk=32, max_batch=4, max_tokens=256, watermark_permille=500, admission="optimistic", groups=[(16, 0, 12)])
    _, acts, _ = run(cfg, {0: [(1, 30, 60), (2, 30, 60), (3, 30, 60)]}, 200)
    assert any(a.preempted for a in acts)
    assert sorted(rid for a in acts for rid in a.finished) == [1, 2, 3]


def test_cancel_blocks_same_tick_arrival_and_frees_a_running_request():
    cfg = SchedConfig(token_budget=32, max_chunk=16, max_batch=4, max_tokens=128, groups=[(16, 0, 16)])
    sched = Scheduler(cfg)
    act = sched.step(SchedInput([(1, 8, 4), (2, 8, 4)], [2], [], [16]))
    assert act.arrival_status == [1, 2] and act.prefill == [(1, 0, 8)]
    act = sched.step(SchedInput([], [1], [], [16]))
    assert act.tokens() == 0 and sched.counts()["live"] == 0


def test_engine_reported_completion_removes_the_request():
    cfg = SchedConfig(token_budget=32, max_chunk=16, max_batch=4, max_tokens=128, groups=[(16, 0, 16)])
    sched = Scheduler(cfg)
    sched.step(SchedInput([(1, 8, 40)], [], [], [16]))
    assert sched.step(SchedInput([], [], [], [15])).decode == [1]
    assert sched.step(SchedInput([], [], [1], [16])).tokens() == 0
    assert sched.request(1) is None


def test_latency_guard_lets_a_starved_request_jump_the_waiting_queue():
    cfg = SchedConfig(token_budget=8, max_chunk=8, max_batch=4, max_tokens=512, max_wait_ticks=3, groups=[(16, 0, 64)])
    sched, acts, _ = run(cfg, {0: [(1, 200, 2)], 1: [(2, 8, 2)]}, 12)
    served2 = [i for i, a in enumerate(acts) if any(p[0] == 2 for p in a.prefill)]
    assert served2 and served2[0] <= 1 + 3 + 1, "request 2 is served once it has waited max_wait_ticks"
    before = acts[served2[0] - 1]
    assert all(p[0] == 1 for p in before.prefill)


def test_windowed_group_counts_only_live_pages():
    cfg = SchedConfig(token_budget=64, max_chunk=16, max_batch=2, max_tokens=1024, admission="committed", groups=[(16, 0, 64), (16, 24, 6)])
    sched = Scheduler(cfg)
    sched.can_ever_fit(500, 100)  # (24 + 16) / 16 + 1 = 4 pages at most in the windowed group
    act = sched.step(SchedInput([(1, 500, 100)], [], [], [64, 6]))
    assert act.arrival_status == [1]


def test_trace_round_trip_and_detects_a_changed_line():
    cfg = SchedConfig(token_budget=24, max_chunk=16, max_batch=3, max_tokens=128, admission="optimistic", groups=[(16, 0, 5)])
    assert parse_config(format_config(cfg)) == cfg
    _, _, trace = run(cfg, {0: [(1, 20, 30)], 1: [(2, 33, 10)], 4: [(3, 5, 5)]}, 60, cancels_by_tick={9: [2]})
    assert replay_trace(trace) == []
    lines = trace.splitlines()
    lines[3] = lines[3].replace("K=", "K=9")
    assert len(replay_trace("\n".join(lines))) == 1
    other = SchedConfig(token_budget=24, max_chunk=8, max_batch=3, max_tokens=128, admission="optimistic", groups=[(16, 0, 5)])
    lines[0] = format_config(other)
    lines[3] = trace.splitlines()[3]
    assert replay_trace("\n".join(lines)), "a different policy must give different decisions"


@pytest.mark.parametrize("seed", range(4))
def test_random_load_keeps_the_invariants(seed):
    rng = np.random.default_rng(seed)
    cfg = SchedConfig(token_budget=int(rng.integers(8, 40)), max_chunk=int(rng.integers(4, 32)), max_batch=6, max_tokens=160,
                      watermark_permille=int(rng.choice([700, 1000])), max_wait_ticks=4, admission="optimistic", groups=[(16, 0, 14)])
    arrivals, rid = {}, 0
    for t in range(0, 120, 3):
        arrivals[t] = []
        for _ in range(int(rng.integers(0, 3))):
            rid += 1
            arrivals[t].append((rid, int(rng.integers(1, 90)), int(rng.integers(1, 40))))
    sched, acts, trace = run(cfg, arrivals, 900)
    done = sorted(r for a in acts for r in a.finished)
    assert done == list(range(1, rid + 1)), "every request finishes"
    assert sched.counts()["live"] == 0
    assert replay_trace(trace) == []


def test_no_cache_group_means_admission_by_slots_alone():
    """A model whose layers keep fixed-size state only has no page group: no
    page is booked, nothing is preempted, and requests are admitted while a
    slot is free, under either admission rule."""
    for admission in ("committed", "optimistic"):
        cfg = SchedConfig(token_budget=64, max_chunk=32, max_batch=2, max_tokens=4096, admission=admission, groups=[])
        s = Scheduler(cfg)
        s.can_ever_fit(4000, 96)
        act = s.step(SchedInput([(1, 40, 3), (2, 3000, 2), (3, 5, 1)], [], [], []))
        assert act.arrival_status == [1, 1, 0]  # two slots
        assert [p[0] for p in act.prefill] == [1, 2] and act.preempted == []
        seen = set()
        for _ in range(200):
            act = s.step(SchedInput([(3, 5, 1)] if 3 not in seen else [], [], [], []))
            if act.arrival_status == [1]:
                seen.add(3)
            assert act.preempted == []
            if not s.counts()["live"] and 3 in seen:
                break
        assert 3 in seen and s.counts()["live"] == 0
        text = format_config(cfg)
        assert text.endswith("G=-") and parse_config(text).groups == []


# -- the reference's recorded runs ---------------------------------------------------
def replay_reference_fixture(fixture: dict, admission: str):
    """Feed a recorded run of the reference's scheduler to ours.  The reference
    keeps a block count of its own (finished requests' blocks stay held as its
    prefix cache until the engine reports them freed, `R=`); ours is told the
    free pages each tick, so the harness keeps that book: pages of live
    requests from our own decisions, plus the blocks the reference would hold
    cached.  `max_new` is translated: the reference counts decode ticks, ours
    counts tokens and the step that ends a prompt yields the first, so the
    reference's max_new is ours plus one.  Returns per tick (ours, reference)
    as (prompt portions, decoded, preempted, finished by the scheduler)."""
    cfg = fixture["cfg"]
    bs, cap = cfg["s"], cfg["k"]
    blocks = lambda n: 0 if n <= 0 else -(-n // bs)
    sched = Scheduler(SchedConfig(token_budget=cfg["b"], max_chunk=cfg["c"], max_batch=32, max_tokens=1 << 20, watermark_permille=cfg["w"],
                                  max_wait_ticks=cfg["t"], admission=admission, groups=[(bs, 0, cap)]))
    live, sizes, cached, deferred, out = {}, {}, 0, [], []
    for tick in fixture["ticks"]:
        cached -= tick["R"]
        for rid in tick["C"]:
            live.pop(rid, None)
        for rid in tick["F"]:
            if rid in live:
                cached += blocks(sum(sizes[rid]))
                live.pop(rid)
        arrivals = deferred + [(i, p, m + 1) for i, p, m in tick["A"] if i not in tick["C"]]
        sizes.update({i: (p, m) for i, p, m in tick["A"]})
        held = sum(blocks(n) for n in live.values())
        act = sched.step(SchedInput(arrivals, tick["C"], tick["F"], [cap - held - cached]))
        deferred = [a for a, status in zip(arrivals, act.arrival_status) if status == 0]
        for rid in act.preempted:
            live[rid] = 0
        for rid, _, end in act.prefill:
            live[rid] = end
        for rid in act.decode:
            live[rid] = live.get(rid, 0) + 1
        for rid in act.finished:
            cached += blocks(sum(sizes[rid]))
            live.pop(rid, None)
        ours = ([list(p) for p in act.prefill], list(act.decode), list(act.preempted), list(act.finished))
        ref = (tick["P"], tick["D"], tick["X"], [f for f in tick["Fout"] if f not in tick["F"]])  # the reference echoes engine-reported completions
        out.append((ours, ref))
    return out, sched


def reference_fixtures():
    import json
    from pathlib import Path

    return json.loads((Path(__file__).parent / "golden" / "scheduler_fixtures.json").read_text())


@pytest.mark.parametrize("admission", ["committed", "optimistic"])
@pytest.mark.parametrize("name", ["s01_long_prompt", "s03_budget_exhausted", "s04_zero_budget", "s05_cancel_race"])
def test_reference_runs_that_ours_decides_the_same(name, admission):
    """Chunked prefill under one token budget, decode before prefill, one
    portion per request per tick, the first token with the last portion, a zero
    budget, cancels that block a same-tick arrival, completions the engine
    reports: every tick's portions, decoded requests, preemptions and finishes
    are the reference's."""
    ticks, _ = replay_reference_fixture(reference_fixtures()[name], admission)
    for t, (ours, ref) in enumerate(ticks, 1):
        assert ours == ref, f"{name} tick {t}: ours {ours} reference {ref}"


def test_reference_run_where_waiting_order_differs_on_purpose():
    """s07_cache_freed: the reference walks waiting requests in slot order, and
    a new arrival takes the lowest free slot, so at tick 3 request 3 (new, in
    the slot request 1 left) goes before request 2, which still owes one prompt
    token.  Ours walks them in admission order: 2 ends its prompt first.  Ticks
    3 to 5 differ by exactly that exchange; every other tick is the same, and
    both finish every request."""
    ticks, sched = replay_reference_fixture(reference_fixtures()["s07_cache_freed"], "committed")
    differ = [t for t, (ours, ref) in enumerate(ticks, 1) if ours != ref]
    assert differ == [3, 4, 5]
    assert ticks[2][0][0] == [[2, 15, 16], [3, 0, 15]] and ticks[2][1][0] == [[3, 0, 16]]
    finished = lambda side: sorted(r for tick in ticks for r in tick[side][3])
    assert finished(0) == finished(1) == [1, 2, 3, 4, 5, 6, 7, 8]
    assert sched.counts()["live"] == 0


@pytest.mark.parametrize("name, first", [("s02_preempt_storm", 9), ("s06_kv_watermark", 13)])
def test_reference_runs_that_storm_where_ours_defers(name, first):
    """Three requests arrive that fit under the watermark only if the blocks of
    earlier, finished requests (still held as the reference's prefix cache) are
    not counted.  The reference admits by the live requests' lengths alone,
    prefills all three and then preempts tick after tick, dozens of times (its
    scenario is named for that).  Ours counts every held page (one book):
    with optimistic admission the arrival that does not fit is deferred at that
    tick, nothing is ever preempted, and every request finishes.  Every tick
    before the arrival is the reference's."""
    fixture = reference_fixtures()[name]
    ticks, sched = replay_reference_fixture(fixture, "optimistic")
    differ = [t for t, (ours, ref) in enumerate(ticks, 1) if ours != ref]
    assert differ[0] == first and all(ours == ref for ours, ref in ticks[: first - 1])
    ours_first, ref_first = ticks[first - 1]
    assert len(ours_first[0]) == 1 and len(ref_first[0]) == 2  # one prompt started where the reference starts two
    assert fixture["ticks"][-1]["preempt_total"] > 30 and all(not ours[2] for ours, _ in ticks)
    arrived = sorted(a[0] for tick in fixture["ticks"] for a in tick["A"])
    assert sorted(r for ours, _ in ticks for r in ours[3]) == arrived and sched.counts()["live"] == 0
