"""The generation loop's decisions (no GPU), driven with a scripted model."""
import pytest

from etalii.dllm_b200.engine.generate import (BatchRun, ContextLengthError, GenerationResult, check_prompts,
                                              plan_batches, run_batches)


def test_plan_batches_fits_pages_and_slots():
    assert plan_batches([10, 10, 10], 10, 1000, 64, 100, 8) == [[0, 1, 2]]
    assert plan_batches([10, 10, 10], 10, 1000, 64, 2, 8) == [[0, 1], [2]]
    assert plan_batches([10] * 5, 10, 1000, 64, 100, 8, max_batch=2) == [[0, 1], [2, 3], [4]]
    assert plan_batches([100, 10], 1000, 128, 64, 3, 8) == [[0], [1]]  # a sequence is capped by the window
    with pytest.raises(ContextLengthError):
        plan_batches([100], 100, 1000, 64, 2, 8)


def test_check_prompts():
    check_prompts([[1, 2], [3]], 10, 5)
    with pytest.raises(ContextLengthError, match="5 tokens; the context window holds 5"):
        check_prompts([[1] * 5], 10, 5)
    with pytest.raises(ValueError, match="outside the vocabulary"):
        check_prompts([[1, 10]], 10, 5)
    with pytest.raises(ValueError, match="empty"):
        check_prompts([[]], 10, 5)


def test_batch_run_rules():
    run = BatchRun([3, 5, 2], max_new_tokens=3, stop_ids=frozenset({9}), context_length=7)
    assert run.active == [0, 1, 2]
    assert run.accept([4, 9, 4]) == [1]           # a stop token ends its sequence and is not output
    assert run.active == [0, 2]
    assert run.accept([5, 5]) == []
    assert run.accept([6, 9]) == [0, 2]           # max_new_tokens reached; a late stop token
    results = run.results()
    assert [r.tokens for r in results] == [(4, 5, 6), (), (4, 5)]
    assert [r.finish_reason for r in results] == ["length", "stop", "stop"]
    assert [r.prompt_tokens for r in results] == [3, 5, 2]
    window = BatchRun([5], max_new_tokens=10, stop_ids=frozenset(), context_length=7)
    assert window.accept([1]) == [] and window.accept([1]) == [0]  # the context is full at 7 tokens
    assert window.results()[0].finish_reason == "length" and len(window.results()[0].tokens) == 2
    nothing = BatchRun([4], max_new_tokens=0, stop_ids=frozenset(), context_length=9)
    assert nothing.active == [] and nothing.results()[0] == GenerationResult((), 4, "length")


def test_fingerprint_is_the_hash_of_int32_ids():
    import hashlib

    result = GenerationResult((1, 2, 300), 2, "stop")
    assert result.fingerprint == hashlib.sha256(bytes([1, 0, 0, 0, 2, 0, 0, 0, 44, 1, 0, 0])).hexdigest()


class Scripted:
    """A stand-in for the device side: a sequence answers (last fed token + 1); records what it was asked."""

    def __init__(self):
        self.open, self.log, self.next_handle = {}, [], 0

    def start(self, indices):
        self.next_handle += 1
        self.open[self.next_handle] = set(range(len(indices)))
        return self.next_handle

    def prefill(self, handle, positions, prompts):
        assert set(positions) <= self.open[handle]
        self.log.append(("prefill", handle, list(positions), [len(p) for p in prompts]))
        return [p[-1] + 1 for p in prompts]

    def decode(self, handle, positions, last, steps):
        assert set(positions) <= self.open[handle] and steps >= 1
        self.log.append(("decode", handle, list(positions), steps))
        return [[t + 1 + k for t in last] for k in range(steps)]

    def finish(self, handle, positions):
        for p in (positions if positions is not None else list(self.open[handle])):
            self.open[handle].remove(p)  # KeyError if something is given back twice


def _run(prompts, batches, fake, max_new, stops, window=100, chunk=16, free_chunk=None):
    def make_run(indices):
        return BatchRun([len(prompts[i]) for i in indices], max_new, frozenset(stops), window)

    return run_batches(prompts, batches, make_run, fake.start, fake.prefill, fake.decode, fake.finish, chunk=chunk,
                       free_chunk=free_chunk)


def test_a_batch_without_stop_tokens_decodes_in_longer_runs():
    """Without stop tokens only the lengths end sequences, and those are known: the host need not look in between.
    With stop tokens the runs stay short, whatever the longer limit is."""
    prompts = [[1, 2, 3], [10]]
    fake = Scripted()
    results = _run(prompts, [[0, 1]], fake, 41, set(), chunk=4, free_chunk=32)
    assert [entry[3] for entry in fake.log if entry[0] == "decode"] == [32, 8]
    assert [len(r.tokens) for r in results] == [41, 41] and results[0].tokens[:3] == (4, 5, 6)
    fake = Scripted()
    _run(prompts, [[0, 1]], fake, 41, {1000}, chunk=4, free_chunk=32)
    assert [entry[3] for entry in fake.log if entry[0] == "decode"] == [4] * 10
    fake = Scripted()
    _run(prompts, [[0, 1]], fake, 41, set(), window=30, chunk=4, free_chunk=32)   # the context ends the first sooner
    assert [entry[3] for entry in fake.log if entry[0] == "decode"][0] == 26


@pytest.mark.parametrize("chunk", [1, 2, 16])
def test_run_batches_shorter_requests_end_earlier_and_everything_is_given_back(chunk):
    prompts = [[10, 11], [20], [30, 31, 32], [40]]
    fake = Scripted()
    results = _run(prompts, [[0, 1], [2, 3]], fake, 4, {23, 42}, chunk=chunk)
    assert [r.tokens for r in results] == [(12, 13, 14, 15), (21, 22), (33, 34, 35, 36), (41,)]
    assert [r.finish_reason for r in results] == ["length", "stop", "length", "stop"]
    assert all(not left for left in fake.open.values())
    assert fake.log[0] == ("prefill", 1, [0, 1], [2, 1])
    if chunk == 1:  # one token each per step, and only for sequences still running
        assert fake.log[1:4] == [("decode", 1, [0, 1], 1), ("decode", 1, [0, 1], 1), ("decode", 1, [0], 1)]
    else:  # never more steps in a run than every active sequence may still take
        assert all(entry[3] <= 3 for entry in fake.log if entry[0] == "decode")


def test_zero_max_tokens_runs_nothing():
    fake = Scripted()
    results = _run([[1, 2], [3]], [[0, 1]], fake, 0, set())
    assert [r.tokens for r in results] == [(), ()] and fake.log == []
    assert all(not left for left in fake.open.values())


def test_run_batches_gives_back_on_error():
    fake = Scripted()

    def failing(handle, positions, prompts):
        raise RuntimeError("device lost")

    with pytest.raises(RuntimeError):
        run_batches([[1], [2]], [[0, 1]], lambda ix: BatchRun([1, 1], 2, frozenset(), 10), fake.start, failing,
                    fake.decode, fake.finish)
    assert all(not left for left in fake.open.values())


def test_kernel_choice_rules_for_products():
    """Which kernel a bfloat16 product takes, as plain functions of its sizes (no device needed)."""
    from etalii.dllm_b200.kernels import ops

    assert ops.streams(1, 128256) and ops.streams(16, 49152)          # up to 16 rows: always streamed
    assert ops.streams(32, 3072) and not ops.streams(32, 49152)       # 17 to 32 rows: unless the matrix is wide
    assert ops.streams(64, 576) and not ops.streams(64, 3072)         # 33 to 64 rows: only narrow matrices
    assert not ops.streams(65, 576)
    # small weights with 17 to 64 rows: the reduction split over a cluster, whatever the number of weight rows
    assert ops.streams(64, 3072, 576) and ops.splits_over_clusters(17, 3072, 576)
    assert ops.splits_over_clusters(16, 3072, 576) and not ops.splits_over_clusters(16, 576, 576)
    assert not ops.splits_over_clusters(8, 3072, 576) and not ops.splits_over_clusters(64, 16384, 2048)
    assert ops.splits_over_clusters(64, 6144, 4096) and not ops.splits_over_clusters(16, 6144, 4096)  # few rows of W
    assert ops.streams_through_shared_memory(1, 28672, 4096) and not ops.streams_through_shared_memory(8, 28672, 4096)
    assert ops.streams_through_shared_memory(8, 4096, 14336) and not ops.streams_through_shared_memory(9, 4096, 14336)
    assert not ops.streams_through_shared_memory(1, 16384, 2048)      # short rows of W
    assert not ops.streams_through_shared_memory(1, 4096, 4096 + 8)   # a reduction that is no multiple of 64
    # a narrow W with a long reduction and 33 to 64 rows: the reduction is cut so that every multiprocessor reads
    assert ops.reduction_split(64, 4096, 14336) == 8 and ops.reduction_split(64, 2048, 8192) == 8
    assert ops.reduction_split(48, 4096, 4096) == 8 and ops.reduction_split(33, 576, 1536) == 1
    assert ops.reduction_split(32, 4096, 14336) == 1 and ops.reduction_split(64, 28672, 4096) == 1
    assert ops.reduction_split(64, 2048, 2048) == 1                   # small: the cluster kernel's
    assert ops.takes_weights_as_rows(64, 28672, 4096) and not ops.takes_weights_as_rows(64, 4096, 14336)
    assert ops.takes_weights_as_rows(16, 28672, 4096) and not ops.takes_weights_as_rows(65, 28672, 4096)
    assert ops.takes_weights_as_rows(3, 28672, 4096) and not ops.takes_weights_as_rows(2, 28672, 4096)
    assert ops.takes_weights_as_rows(9, 16384, 2048) and not ops.takes_weights_as_rows(8, 16384, 2048)
    assert not ops.takes_weights_as_rows(16, 49152, 576) and ops.takes_weights_as_rows(17, 49152, 576)
