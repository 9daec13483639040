"""Hand-derived answers for the attention oracle (oracle/attention_np.py)."""
import numpy as np

from oracle import attention_np as an


def test_uniform_scores_average_the_values():
    q = np.zeros((1, 2, 1, 4))
    k = np.ones((1, 3, 1, 4))
    v = np.arange(12, dtype=np.float64).reshape(1, 3, 1, 4)
    out, lse = an.mha_forward(q, k, v, 0.5, causal=False)
    assert np.allclose(out[0, :, 0], v[0, :, 0].mean(axis=0))      # all scores 0: plain average of the three value rows
    assert np.allclose(lse, np.log(3.0))                           # max 0 + log(sum of three ones)


def test_causal_mask_is_aligned_to_the_bottom_right():
    # two queries against three keys: row 0 sees keys 0, 1; row 1 sees keys 0, 1, 2
    q = np.zeros((1, 2, 1, 2))
    k = np.zeros((1, 3, 1, 2))
    v = np.array([[1.0, 0], [3.0, 0], [8.0, 0]]).reshape(1, 3, 1, 2)
    out, lse = an.mha_forward(q, k, v, 1.0, causal=True)
    assert np.allclose(out[0, 0, 0], [2.0, 0]) and np.allclose(out[0, 1, 0], [4.0, 0])
    assert np.allclose(lse[0, 0], [np.log(2.0), np.log(3.0)])


def test_more_queries_than_keys_leaves_early_rows_empty():
    q = np.zeros((1, 3, 1, 2))
    k = np.zeros((1, 1, 1, 2))
    v = np.full((1, 1, 1, 2), 5.0)
    out, lse = an.mha_forward(q, k, v, 1.0, causal=True)
    assert (out[0, :2] == 0).all() and np.isinf(lse[0, 0, :2]).all()   # rows 0 and 1 see nothing: zeros, lse = +inf
    assert np.allclose(out[0, 2, 0], 5.0) and np.isclose(lse[0, 0, 2], 0.0)


def test_softmax_known_values_and_grouped_heads():
    # scores (1, 2, 3) through a scale of 1: the literals of the reference's softmax test (reduce_test.go:1665-1717)
    q = np.array([1.0, 0]).reshape(1, 1, 1, 2).repeat(2, axis=2)   # two query heads sharing one kv head
    k = np.array([[1.0, 0], [2.0, 0], [3.0, 0]]).reshape(1, 3, 1, 2)
    v = np.eye(3)[:, :2].reshape(1, 3, 1, 2)
    out, _ = an.mha_forward(q, k, v, 1.0, causal=False)
    assert np.allclose(out[0, 0, 0], [0.09003057, 0.24472848], atol=1e-7)
    assert np.allclose(out[0, 0, 1], out[0, 0, 0])


def test_bf16_round_trip():
    x = np.array([1.0, 1.00390625, -3.1415926, 65504.0, 1e-8], dtype=np.float32)
    back = an.from_bf16_bits(an.to_bf16_bits(x))
    assert back[0] == 1.0 and abs(back[2] + 3.140625) < 1e-6 and np.all(np.abs(back - x) <= np.abs(x) * 2 ** -8)
