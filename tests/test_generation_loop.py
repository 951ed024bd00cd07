"""The generation loop's decisions with a fake backend (no GPU).

The fake plays the part of the reference's `SequenceModel` (crates/engine/src/model_engine/
tests/mod.rs:19-128): it returns fixed logits that depend on the position, records every
step, and can be told to fail.
"""
import pytest

from tau_rs_b200.engine import GenerationMetrics, generate_tokens, plan_batches


class FakeBackend:
    """The next token after position `p` of request content `c` is `(c + p) % vocab`, where `c` is the first prompt token."""

    def __init__(self, capacity_tokens=64 * 8, max_sequence_tokens=256, vocab=50, fail_at_step=None):
        self.capacity_tokens, self.max_sequence_tokens, self.vocab = capacity_tokens, max_sequence_tokens, vocab
        self.free = list(range(16))[::-1]
        self.open, self.lengths, self.first = set(), {}, {}
        self.steps, self.opened, self.closed = [], [], []
        self.fail_at_step = fail_at_step

    def open_sequence(self):
        slot = self.free.pop()
        self.open.add(slot)
        self.lengths[slot] = 0
        self.opened.append(slot)
        return slot

    def close_sequence(self, slot):
        assert slot in self.open, "closed twice"
        self.open.remove(slot)
        self.free.append(slot)
        self.closed.append(slot)

    def step(self, entries):
        if self.fail_at_step is not None and len(self.steps) == self.fail_at_step:
            raise RuntimeError("injected failure")
        self.steps.append([(entry.slot, self.lengths[entry.slot], len(entry.tokens), tuple(entry.want)) for entry in entries])
        rows = []
        for entry in entries:
            assert entry.slot in self.open
            if self.lengths[entry.slot] == 0:
                self.first[entry.slot] = entry.tokens[0]
            for place in entry.want:
                rows.append((self.first[entry.slot] + self.lengths[entry.slot] + place) % self.vocab)
            self.lengths[entry.slot] += len(entry.tokens)
        return rows


def select(rows, request_ids, token_indices):
    select.calls.append((list(request_ids), list(token_indices)))
    return list(rows)


@pytest.fixture(autouse=True)
def reset_select():
    select.calls = []


def expected_tokens(prompt, count, vocab=50):
    return [(prompt[0] + len(prompt) - 1 + index) % vocab for index in range(count)]


def test_offsets_chunks_and_the_limit():
    """A 10-token prompt in chunks of 4: steps start at 0, 4, 8, then decode at 10, 11, 12; only the
    last chunk is sampled; the first token counts toward the limit (tests/generation.rs:48-125,213-243)."""
    backend = FakeBackend()
    metrics = GenerationMetrics()
    (result,) = generate_tokens(backend, [[5] * 10], 4, select, prefill_chunk_tokens=4, metrics=metrics)
    assert [step[0][1:] for step in backend.steps] == [(0, 4, ()), (4, 4, ()), (8, 2, (1,)), (10, 1, (0,)), (11, 1, (0,)), (12, 1, (0,))]
    assert result.tokens == expected_tokens([5] * 10, 4) and result.finish_reason == "length" and result.prompt_tokens == 10
    assert select.calls[0] == ([0], [0]) and select.calls[-1] == ([0], [3])
    assert (metrics.prompt_tokens, metrics.generated_tokens, metrics.decode_tokens, metrics.prefill_steps, metrics.decode_steps) == (10, 4, 3, 3, 3)
    assert backend.open == set() and backend.opened == backend.closed


def test_stop_token_after_the_prompt_means_no_decode_step():
    backend = FakeBackend()
    (result,) = generate_tokens(backend, [[7, 1, 1]], 5, select, stop_tokens=[9])
    assert result.tokens == [] and result.finish_reason == "stop" and len(backend.steps) == 1 and backend.open == set()


def test_stop_token_is_neither_returned_nor_fed_back():
    backend = FakeBackend()
    (result,) = generate_tokens(backend, [[7, 1, 1]], 8, select, stop_tokens=[12])
    assert result.tokens == [9, 10, 11] and result.finish_reason == "stop"
    assert sum(step[0][2] for step in backend.steps) == 3 + 3     # the prompt and the three tokens that were kept


def test_zero_limit_touches_nothing_and_bad_requests_are_refused():
    backend = FakeBackend()
    results = generate_tokens(backend, [[1, 2], []], [0, 0], select)
    assert [r.tokens for r in results] == [[], []] and [r.finish_reason for r in results] == ["length", "length"]
    assert backend.steps == [] and backend.opened == []
    for prompts, limits in [([[]], 3), ([[1] * 250], 10), ([[1]], -1)]:
        with pytest.raises(ValueError):
            generate_tokens(backend, prompts, limits, select)
    with pytest.raises(ValueError):
        generate_tokens(backend, [[1]], 1, select, prefill_chunk_tokens=0)
    assert backend.steps == []


def test_unequal_batch_shorter_requests_end_earlier_and_order_is_kept():
    backend = FakeBackend()
    prompts = [[3] * 5, [8] * 11, [20] * 17]
    results = generate_tokens(backend, prompts, [2, 6, 4], select)
    for prompt, limit, result in zip(prompts, [2, 6, 4], results):
        assert result.tokens == expected_tokens(prompt, limit)
    assert [len(step) for step in backend.steps] == [3, 3, 2, 2, 1, 1]     # prefill, then the batch shrinks
    assert backend.closed[0] == backend.opened[0] and backend.open == set()


def test_more_requests_than_fit_run_batch_after_batch_on_the_same_slots():
    backend = FakeBackend(capacity_tokens=64 * 3)
    prompts = [[index + 1] * (index + 2) for index in range(7)]
    metrics = GenerationMetrics()
    results = generate_tokens(backend, prompts, 3, select, max_batch=4, metrics=metrics)
    assert [result.tokens for result in results] == [expected_tokens(prompt, 3) for prompt in prompts]
    assert metrics.batches == 3 and set(backend.opened) == {0, 1, 2}       # three pages of 64 tokens: three requests at a time
    assert plan_batches([10, 70, 10, 10, 200], max_batch=2, capacity_tokens=256) == [[0, 1], [2, 3], [4]]
    with pytest.raises(ValueError):
        plan_batches([300], max_batch=2, capacity_tokens=256)


def test_slots_are_given_back_when_a_step_fails():
    for failing in (0, 1, 3):
        backend = FakeBackend(fail_at_step=failing)
        with pytest.raises(RuntimeError):
            generate_tokens(backend, [[1] * 6, [2] * 3], 5, select, prefill_chunk_tokens=6)
        assert backend.open == set() and sorted(backend.opened) == sorted(backend.closed)
        backend.fail_at_step = None
        assert generate_tokens(backend, [[4, 4]], 2, select)[0].tokens == expected_tokens([4, 4], 2)   # no retry needed, the next request works


# ---- one step ahead of the host ---------------------------------------------------------------------
class AheadBackend(FakeBackend):
    """Also takes the tokens of a step from "the device" (here: a list that the fake `launch` handed out)."""
    accepts_device_tokens = True

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.from_device = []

    def step(self, entries, device_tokens=None):
        if device_tokens is not None:
            assert len(device_tokens) == len(entries) and all(len(entry.tokens) == 1 for entry in entries)
            self.from_device.append(list(device_tokens))
        return super().step(entries)


class Handle:
    def __init__(self, rows):
        self.tokens = list(rows)


class TwoHalves:
    """A `select` in two halves; `collected` counts how many steps the host has seen the tokens of."""

    def __init__(self):
        self.launched, self.collected, self.order = 0, 0, []

    def launch(self, rows, request_ids, token_indices):
        self.launched += 1
        self.order.append(("launch", list(request_ids), list(token_indices)))
        return Handle(rows)

    def collect(self, handle):
        self.collected += 1
        self.order.append(("collect",))
        return list(handle.tokens)

    def __call__(self, rows, request_ids, token_indices):
        return self.collect(self.launch(rows, request_ids, token_indices))


@pytest.mark.parametrize("stop", [(), (9,), (7, 30)])
def test_one_step_ahead_gives_the_same_tokens_and_reasons(stop):
    prompts = [[3, 4, 5], [20], [7] * 10, [41, 2]]
    limits = [6, 1, 12, 4]
    plain = generate_tokens(FakeBackend(), prompts, limits, select, stop_tokens=stop)
    backend, halves = AheadBackend(), TwoHalves()
    ahead = generate_tokens(backend, prompts, limits, halves, stop_tokens=stop)
    assert [(r.tokens, r.finish_reason) for r in ahead] == [(r.tokens, r.finish_reason) for r in plain]
    assert not backend.open and sorted(backend.closed) == sorted(backend.opened)      # every slot given back once


def test_one_step_ahead_starts_the_next_step_before_it_reads_the_last():
    backend, halves = AheadBackend(), TwoHalves()
    results = generate_tokens(backend, [[1, 2], [5]], [4, 2], halves)
    assert [r.tokens for r in results] == [expected_tokens([1, 2], 4), expected_tokens([5], 2)]
    # After the prefill (one launch and its collect): launch of decode step 1, launch of step 2, then the collect of step 1.
    decode = halves.order[2:]
    assert [event[0] for event in decode[:3]] == ["launch", "launch", "collect"]
    # Request 1 reaches its limit of 2 with the token of decode step 1: it is not in step 2.
    assert decode[0][1] == [0, 1] and decode[1][1] == [0]
    # Token indices: the token being chosen is one further than what the host has booked.
    assert decode[0][2] == [1, 1] and decode[1][2] == [2]
    assert len(backend.from_device) == 2 and all(len(tokens) == 1 for tokens in backend.from_device)


def test_one_step_ahead_drops_the_token_computed_past_a_stop():
    # Request 0 yields 3, 4, 5, ...; 5 is a stop token.  Its step after the 5 has been started already and is thrown away.
    backend, halves = AheadBackend(), TwoHalves()
    results = generate_tokens(backend, [[1, 2, 3], [10]], [8, 8], halves, stop_tokens=(5,))
    assert results[0].tokens == [3, 4] and results[0].finish_reason == "stop"
    assert results[1].tokens == expected_tokens([10], 8) and results[1].finish_reason == "length"
    slot0_steps = [step for step in backend.steps if any(entry[0] == backend.opened[0] for entry in step)]
    assert len(slot0_steps) == 1 + 3       # the prompt, the steps fed 3 and 4, and the one fed 5 for nothing


def test_one_step_ahead_equals_step_by_step_on_random_requests():
    """Many random mixes of prompts, limits, stop tokens, batch sizes and prefill chunks: the loop that runs ahead returns what
    the plain loop returns, gives every slot back once, and never steps a request that has ended."""
    import random

    rng = random.Random(7)
    for trial in range(200):
        count = rng.randint(1, 7)
        prompts = [[rng.randrange(50) for _ in range(rng.randint(1, 12))] for _ in range(count)]
        limits = [rng.randint(0, 9) for _ in range(count)]
        stop = tuple(rng.sample(range(50), rng.randint(0, 6)))
        max_batch = rng.randint(1, 4)
        chunk = rng.choice([None, 1, 3, 8])
        plain = generate_tokens(FakeBackend(), prompts, limits, select, stop_tokens=stop, max_batch=max_batch, prefill_chunk_tokens=chunk)
        backend, metrics = AheadBackend(), GenerationMetrics()
        ahead = generate_tokens(backend, prompts, limits, TwoHalves(), stop_tokens=stop, max_batch=max_batch, prefill_chunk_tokens=chunk,
                                metrics=metrics)
        assert [(r.tokens, r.finish_reason, r.prompt_tokens) for r in ahead] == [(r.tokens, r.finish_reason, r.prompt_tokens) for r in plain], trial
        assert not backend.open and sorted(backend.closed) == sorted(backend.opened)
        assert metrics.generated_tokens == sum(len(r.tokens) for r in ahead)


def test_prompt_file_takes_json_or_lines(tmp_path):
    from tau_rs_b200.cli import read_prompt_file

    as_json = tmp_path / "prompts.json"
    as_json.write_text("[[5, 6, 7], [8, 9]]\n")
    assert read_prompt_file(str(as_json)) == [[5, 6, 7], [8, 9]]
    as_lines = tmp_path / "prompts.txt"
    as_lines.write_text("5 6 7\n\n8,9\n 10, 11 \n")
    assert read_prompt_file(str(as_lines)) == [[5, 6, 7], [8, 9], [10, 11]]
    for bad in ("[[1, 2], []]", "[1, 2]", "[[1.5]]", "1 two 3\n", "[[1, 2]"):
        wrong = tmp_path / "wrong"
        wrong.write_text(bad)
        with pytest.raises(SystemExit, match="prompt-file"):
            read_prompt_file(str(wrong))


def test_vram_sampler_keeps_start_peak_end_and_a_failed_sample():
    """The record of `--vram-metrics`: crates/metrics/src/memory.rs:47-64 (peak over the samples, delta against the start,
    an error kept even if later samples succeed)."""
    import io
    import json
    import time

    from tau_rs_b200 import vram

    values = iter([100, 180, RuntimeError("query failed"), 260, 150, 120])
    taken = []

    def sample():
        value = next(values, 120)
        taken.append(value)
        if isinstance(value, Exception):
            raise value
        return value

    sampler = vram.VramSampler(sample, "process_on_device", "GPU-0000", interval_ms=5).start()
    while len(taken) < 5:
        time.sleep(0.005)
    snapshot = sampler.finish()
    assert snapshot["vram_start_bytes"] == 100 and snapshot["vram_peak_sampled_bytes"] == 260
    assert snapshot["vram_end_bytes"] in (150, 120) and snapshot["vram_peak_delta_bytes"] == 160
    assert snapshot["vram_error"] == "query failed" and snapshot["vram_samples"] == len(taken) - 1
    assert snapshot["vram_sample_interval_ms"] == 5 and snapshot["vram_scope"] == "process_on_device"
    out = io.StringIO()
    line = vram.report(snapshot, "folder", request_id=3, stream=out)
    assert line.startswith("inference_vram_metrics ") and out.getvalue().strip() == line
    record = json.loads(line.split(" ", 1)[1])
    assert record["request_id"] == 3 and record["model"] == "folder" and record["status"] == "ok" and record["error"] is None
    assert record["vram_peak_sampled_bytes"] == 260 and record["vram_device_uuid"] == "GPU-0000"
    failed = json.loads(vram.report(snapshot, "folder", error="out of pages", stream=out).split(" ", 1)[1])
    assert failed["status"] == "error" and failed["error"] == "out of pages"
    never = vram.VramSampler(lambda: (_ for _ in ()).throw(RuntimeError("no device")), "device", None, interval_ms=5).start().finish()
    assert never["vram_start_bytes"] is None and never["vram_peak_delta_bytes"] is None and never["vram_error"] == "no device"


def test_metrics_send_a_progress_record_when_one_is_due():
    """crates/metrics/src/serving.rs:92-95,160-165: checked at token boundaries, every 5 s; the interval's rate is the
    decode work since the record before (:118-121), the request's rate is over all of it."""
    records = []
    metrics = GenerationMetrics(log_interval_s=5.0, sink=records.append)
    begin = metrics._started
    metrics.decode_tokens, metrics.decode_ms = 10, 1000.0
    metrics.tick(begin + 1.0)
    assert records == []
    metrics.tick(begin + 5.5)
    assert len(records) == 1 and records[0]["status"] == "running" and records[0]["decode_tokens_per_second"] == 10.0
    assert records[0]["interval_decode_tokens_per_second"] == 10.0 and records[0]["elapsed_ms"] == 5500.0
    metrics.decode_tokens, metrics.decode_ms = 40, 2000.0
    metrics.tick(begin + 9.0)                     # 3.5 s after the last record
    assert len(records) == 1
    metrics.tick(begin + 10.6)
    assert records[1]["interval_decode_tokens_per_second"] == 30.0 and records[1]["decode_tokens_per_second"] == 20.0
    final = metrics.report("ok", begin + 11.0)
    assert final["status"] == "ok" and final["interval_decode_tokens_per_second"] is None and final["decode_tokens"] == 40
    silent = GenerationMetrics()
    silent.tick(begin + 100.0)                    # no sink: nothing happens


def test_the_loop_reports_progress_both_ways_of_decoding():
    for ahead in (False, True):
        records = []
        metrics = GenerationMetrics(log_interval_s=0.0, sink=records.append)
        backend = AheadBackend() if ahead else FakeBackend()
        results = generate_tokens(backend, [[1, 2, 3], [4]], 5, TwoHalves() if ahead else select, (), 8, None, metrics)
        assert [result.tokens for result in results] == [expected_tokens([1, 2, 3], 5), expected_tokens([4], 5)]
        assert records and all(record["status"] == "running" for record in records)
        assert records[-1]["decode_tokens"] <= metrics.decode_tokens == 8 and metrics.decode_ms > 0


def test_decode_split_rule_stays_within_what_the_kernel_and_the_machine_take():
    """The number of context blocks of decode attention, for every batch and context and for machines of several sizes:
    at least one block of 64 positions each, never more blocks than are resident at once (four per SM) unless one split
    is all there is, clusters of more than 8 only while they fill at most half of the places, at most 16 in a cluster and
    32 at all; the same for every length of a power-of-two bucket, because a captured graph is keyed by the bucket."""
    from tau_rs_b200.csrc.kernels import decode_splits

    for sms in (148, 132, 16):
        for kv_blocks in (1, 2, 8, 16):
            for n_seqs in (1, 2, 3, 4, 8, 13, 32, 64, 200):
                for length in (1, 2, 63, 64, 65, 200, 1024, 2049, 4096, 8192, 8193, 32001, 131072):
                    splits = decode_splits(n_seqs, length, kv_blocks, sms)
                    blocks = n_seqs * kv_blocks
                    bucket = 1 << max(0, (length - 1).bit_length())
                    assert 1 <= splits <= (16 if bucket <= 8192 else 32)
                    assert splits == 1 or (splits * 64 <= bucket and splits * blocks <= 4 * sms)
                    assert not (8 < splits <= 16) or blocks * splits <= 2 * sms
                    assert not (1 < splits <= 16) or blocks * splits * 100 <= 4 * sms * (98 if splits == 2 else 95 if splits <= 5 else 87)   # clusters leave the last places empty
                    low = bucket // 2 + 1
                    assert decode_splits(n_seqs, low, kv_blocks, sms) == splits == decode_splits(n_seqs, bucket, kv_blocks, sms)
    assert decode_splits(8, 2049, 8, 148) == 8 and decode_splits(1, 2049, 8, 148) == 16 and decode_splits(64, 2049, 8, 148) == 1
    assert decode_splits(8, 2049, 8, 132) == 7 and decode_splits(8, 2049, 8, 74) == 4
    assert [decode_splits(n, 2049, 8, 148) for n in (9, 10, 12, 14, 16, 24, 32, 36, 37)] == [7, 6, 5, 5, 4, 2, 2, 2, 1]


def test_a_row_of_nan_is_an_error_only_for_a_request_that_is_still_going():
    """One step ahead of the host, a request that stopped has one more token computed for nothing; if that row holds
    nothing to choose from (the selector's -1), nobody asked for it.  The same answer for a live request is the
    reference's "model logits are all NaN" (crates/engine/src/generation.rs:81-95)."""
    from tau_rs_b200.config.errors import AllLogitsNaN

    class NaNAfterStop(TwoHalves):
        """Gives -1 for request 0 from its token index 3 on."""

        def launch(self, rows, request_ids, token_indices):
            rows = [-1 if request == 0 and index >= self.first_bad else row for row, request, index in zip(rows, request_ids, token_indices)]
            return super().launch(rows, request_ids, token_indices)

    prompts = [[7, 1, 1], [20, 2]]
    free = [expected_tokens(prompt, 6) for prompt in prompts]
    selector = NaNAfterStop()
    selector.first_bad = 3
    results = generate_tokens(AheadBackend(), prompts, 6, selector, stop_tokens=[free[0][2]])
    assert results[0].tokens == free[0][:2] and results[0].finish_reason == "stop"    # its row of token index 3 was computed and dropped
    assert results[1].tokens == free[1]
    selector = NaNAfterStop()
    selector.first_bad = 2
    backend = AheadBackend()
    with pytest.raises(AllLogitsNaN):
        generate_tokens(backend, prompts, 6, selector, stop_tokens=[free[0][4]])
    assert backend.open == set()
