"""The known-answer vectors the reference's own tests hold next to the path, read from its test sources as text:
`argmaxLast` (tests/test_sampling.nim:4-30), which ends every greedy step of the token-stream checks, and the fp16
bit patterns of `halfToFloat` (tests/test_quant.nim:5-15), the storage format of the KV cache.  (The reference holds
no vector for the attention arithmetic itself: its one golden token stream, tests/integration_inference.nim:15-18,
needs a GGUF model file.)"""
import numpy as np

import oracle
from hippo_leap_b200 import backend as B


def test_argmax_last_golden_cases_of_the_reference():
    # tests/test_sampling.nim:4-10  row-major [1, nVocab]
    assert B.argmaxLast(np.array([[0.1, 0.5, 0.3, 0.9]], np.float32), 4) == 3
    # tests/test_sampling.nim:12-18  column-major [nVocab, 1]
    assert B.argmaxLast(np.array([[0.2], [0.8], [0.1], [0.4]], np.float32), 4) == 1
    # tests/test_sampling.nim:20-30  two positions: the last one decides
    assert B.argmaxLast(np.array([[0.9, 0.1, 0.1, 0.1], [0.1, 0.1, 0.1, 0.8]], np.float32), 4) == 3
    # first maximal index wins (sampling.nim:13-19)
    assert B.argmaxLast(np.array([[0.5, 0.7, 0.7, 0.1]], np.float32), 4) == 1


def test_half_bit_patterns_of_the_reference():
    # tests/test_quant.nim:5-15
    known = {0x0000: 0.0, 0x3C00: 1.0, 0xBC00: -1.0, 0x4000: 2.0, 0x3800: 0.5}
    for bits, value in known.items():
        assert np.array([bits], np.uint16).view(np.float16)[0] == np.float16(value)
        # and the oracle's fp16 rounding (what the fp16-KV variant applies to K and V) keeps these values exactly
        assert oracle.round_fp16(np.array([value], np.float32))[0] == np.float32(value)
    assert np.isposinf(np.array([0x7C00], np.uint16).view(np.float16)[0])
    assert np.isneginf(np.array([0xFC00], np.uint16).view(np.float16)[0])
    assert np.isnan(np.array([0x7C01], np.uint16).view(np.float16)[0])


def test_oracle_matmul_reproduces_the_wmma_known_answers(wmma_known_answers):
    for a, b, c in wmma_known_answers:
        assert np.array_equal(a.astype(np.float16).astype(np.float32), a)
        assert np.array_equal(oracle.matmul(a, b), c)
