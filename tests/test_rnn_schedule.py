"""Token chunking and redirect tables: the three known-answer tests of the reference
(src/runtime/infer/rnn.rs:362-569) replayed through the C ABI.  Pure host logic, no GPU."""
import importlib

wrk = importlib.import_module("web-rwkv_b200")
rt = importlib.import_module("web-rwkv_b200.runtime")

LAST, FULL, NONE = wrk.RNN_LAST, wrk.RNN_FULL, wrk.RNN_NONE


def _input(spec, chunk):
    return rt.RnnInput([([tok] * n, opt) for tok, n, opt in spec], chunk)


def test_run_iter():
    run = _input([(0, 139, LAST), (1, 1, LAST), (2, 0, FULL), (3, 65, FULL)], 128)
    it = run.iter()
    assert it.next() == [(65, NONE), (1, LAST), (0, FULL), (62, FULL)]
    assert it.next() == [(60, NONE), (1, LAST), (0, FULL), (3, FULL)]
    assert it.next() == [(14, LAST), (1, LAST), (0, FULL), (1, FULL)]
    assert it.next() == [(1, LAST), (1, LAST), (0, FULL), (1, FULL)]
    assert it.next() == [(1, LAST), (1, LAST), (0, FULL), (1, FULL)]


def test_advance():
    run = _input([(0, 139, LAST), (1, 1, LAST), (2, 0, FULL), (3, 65, FULL)], 128)
    run.step()
    assert run.iter().next() == [(61, NONE), (0, LAST), (0, FULL), (3, FULL)]
    run = _input([(0, 61, LAST), (1, 1, LAST), (2, 0, FULL), (3, 3, FULL)], 128)
    assert run.iter().next() == [(60, NONE), (1, LAST), (0, FULL), (3, FULL)]


def test_redirect():
    run = _input([(0, 61, LAST), (1, 0, LAST), (2, 0, FULL), (3, 3, FULL)], 128)
    headers, inputs, outputs = rt.redirect(run.iter().next())
    assert headers == [60, 61, 62, 63]
    assert inputs == [(0, 61), (61, 61), (61, 61), (61, 64)]
    assert outputs == [(0, 1), (1, 1), (1, 1), (1, 4)]
    run = _input([(0, 11, LAST), (1, 8, LAST), (2, 9, LAST), (3, 4, LAST)] * 2, 32)
    headers, inputs, outputs = rt.redirect(run.iter().next())
    assert headers == [15, 31]
    assert inputs == [(0, 4), (4, 8), (8, 12), (12, 16), (16, 20), (20, 24), (24, 28), (28, 32)]
    assert outputs == [(0, 0), (0, 0), (0, 0), (0, 1), (1, 1), (1, 1), (1, 1), (1, 2)]


def test_token_chunk_size_is_clamped_and_rounded():
    assert _input([(0, 1, LAST)], 0).token_chunk_size == 32
    assert _input([(0, 1, LAST)], 33).token_chunk_size == 64
    assert _input([(0, 1, LAST)], 256).token_chunk_size == 256


def test_chunks_over_32_round_down_and_decode_continues():
    run = _input([(7, 256, LAST)], 32)
    seen = []
    while run.num_token():
        seen.append(run.iter().next()[0])
        run.step()
    assert seen == [(32, NONE)] * 7 + [(32, LAST)]
    # 139 tokens at chunk 128: one 128-token job, then 11 tokens in one job (11 <= 32 is not rounded)
    run = _input([(7, 139, LAST)], 128)
    assert run.iter().next() == [(128, NONE)]
    run.step()
    assert run.iter().next() == [(11, LAST)]
