"""CPU-only: the C restatement against the known-answer values the reference's own
tests hold for this path (restated here because its gtest binary cannot be built
offline). Each case names the reference test it comes from."""
import numpy as np

import oracle
from oracle import BF16, F32

P = oracle.port()


def test_ones_matmul():  # tests/unified_tests.cpp:50-64: ones[2,3]·ones[3,2] = 3
    assert np.array_equal(P.matmul(np.ones((2, 3), np.float32), np.ones((3, 2), np.float32), F32),
                          np.full((2, 2), 3, np.float32))


def test_batched_matmul_equals_k():  # tests/unified_tests.cpp:235-314: [8,4,16]x[16,32] of ones = 16... K
    a, b = np.ones((8 * 4, 16), np.float32), np.ones((16, 32), np.float32)
    assert np.array_equal(P.matmul(a, b, F32), np.full((32, 32), 16, np.float32))


def test_linear_relu_artifact_values():  # tests/test_inference.cpp:887-919
    w, b = np.array([[1, -1], [0.5, 2]], np.float32), np.array([0.25, -0.75], np.float32)
    assert np.array_equal(P.linear(np.array([[2, 3]], np.float32), w, b, F32, "relu"),
                          np.array([[3.75, 3.25]], np.float32))


def test_linear_diag_values():  # tests/test_inference.cpp:990-1022
    w, b = np.diag([2, 3]).astype(np.float32), np.array([1, -2], np.float32)
    assert np.array_equal(P.linear(np.array([[4, 5]], np.float32), w, b, F32), np.array([[9, 13]], np.float32))


def test_gelu_values():  # tests/test_nn.cpp:385-402: GELU(-2,0,2) ≈ -0.0643, 0, 1.9357 @5e-3
    y = P.activation(np.array([-2, 0, 2], np.float32), F32, "gelu")
    assert np.allclose(y, [-0.0643, 0.0, 1.9357], atol=5e-3)


def test_layer_norm_statistics():  # tests/test_nn.cpp:447-482: rows → mean 0 ±1e-4, var 1 ±2e-3
    rng = np.random.default_rng(0)
    x = (rng.standard_normal((4, 64)) * 3 + 1).astype(np.float32)
    y = P.layer_norm(x, np.ones(64, np.float32), np.zeros(64, np.float32), F32)
    assert np.allclose(y.mean(-1), 0, atol=1e-4) and np.allclose(y.var(-1), 1, atol=2e-3)


def test_global_avg_pool():  # tests/test_nn.cpp:271-290: GAP of [1,2,3,4] = 2.5
    x = np.array([1, 2, 3, 4], np.float32).reshape(1, 1, 2, 2)
    assert P.global_avg_pool(x).reshape(-1)[0] == 2.5


def test_conv_ones():  # tests/unified_tests.cpp:66-82: 3x3 ones * 2x2 ones, no padding → 4
    y = P.conv2d(np.ones((1, 1, 3, 3), np.float32), np.ones((1, 1, 2, 2), np.float32), np.zeros(1, np.float32))
    assert np.array_equal(y, np.full((1, 1, 2, 2), 4, np.float32))


def test_causal_first_token_independent_of_later_tokens():  # tests/test_nn.cpp:594-629
    rng = np.random.default_rng(1)
    E, H, T = 16, 2, 6
    params = []
    for _ in range(4):
        params += [(rng.standard_normal((E, E)) * 0.3).astype(np.float32),
                   (rng.standard_normal(E) * 0.1).astype(np.float32)]
    x1 = rng.standard_normal((1, T, E)).astype(np.float32)
    x2 = x1.copy()
    x2[0, 1:] = rng.standard_normal((T - 1, E)).astype(np.float32)
    y1, y2 = P.mha(x1, params, H, True, F32), P.mha(x2, params, H, True, F32)
    assert np.allclose(y1[0, 0], y2[0, 0], atol=1e-4)


def test_all_reduce_sum():  # tests/test_backend_manager.cpp:1371-1397: [1,2]+[3,4] → [4,6]
    out = P.all_reduce_sum([np.array([1, 2], np.float32), np.array([3, 4], np.float32)], F32)
    assert np.array_equal(out, np.array([4, 6], np.float32))


def test_bf16_matmul_keeps_dtype():  # tests/test_tensor.cpp:157-177
    a = oracle.to_bf16(np.array([[1, 2, 3], [4, 5, 6]], np.float32))
    b = oracle.to_bf16(np.array([[7, 8], [9, 10], [11, 12]], np.float32))
    y = P.matmul(a, b, BF16)
    assert y.dtype == np.uint16 and np.array_equal(oracle.from_bf16(y), [[58, 64], [139, 154]])


def test_bf16_rounding_is_round_to_nearest_even():  # src/types.hpp:311-317
    assert oracle.to_bf16(np.array([1.0 + 2 ** -8], np.float32))[0] == 0x3F80  # tie → even (down)
    assert oracle.to_bf16(np.array([1.0 + 3 * 2 ** -8], np.float32))[0] == 0x3F82  # tie → even (up)
