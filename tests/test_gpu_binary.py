"""GPU: broadcasting binary ops against numpy (float32: bit-exact, one correctly rounded
op per element like the reference CPU kernels; bfloat16: double evaluation rounded to
bf16 like the reference's typed fallback)."""
import numpy as np
import pytest

import oracle
from oracle import BF16, F32
from tests.util import empty_dev, to_dev, to_host

pytestmark = pytest.mark.gpu

OPS = {"add": np.add, "sub": np.subtract, "mul": np.multiply, "div": np.divide}


def elem_strides(shape, out_shape):
    """element strides of a dense tensor of `shape` broadcast to `out_shape` (0 where broadcast)."""
    shape = (1,) * (len(out_shape) - len(shape)) + tuple(shape)
    st, acc = [], 1
    for d in reversed(range(len(shape))):
        st.append(0 if shape[d] == 1 and out_shape[d] != 1 else acc)
        acc *= shape[d]
    return list(reversed(st))


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
@pytest.mark.parametrize("sa,sb", [((64, 48), (64, 48)), ((64, 48), (48,)), ((5, 7, 9), (1,)),
                                   ((3, 1, 8), (1, 6, 8)), ((2, 3, 4, 5, 6, 7), (7,))])
def test_binary_broadcast(dtype, op, sa, sb):
    import munet_b200 as mb
    ctx = mb.Context(0)
    rng = np.random.default_rng(len(sa) * 7 + len(sb))
    a = rng.standard_normal(sa).astype(np.float32)
    b = (rng.standard_normal(sb) + 3.0).astype(np.float32)
    out_shape = np.broadcast_shapes(sa, sb)
    if dtype == BF16:
        ab, bb = oracle.to_bf16(a), oracle.to_bf16(b)
        want = oracle.to_bf16(OPS[op](oracle.from_bf16(ab).astype(np.float64),
                                      oracle.from_bf16(bb).astype(np.float64)).astype(np.float32))
        a_in, b_in = ab, bb
    else:
        want = OPS[op](a, b).astype(np.float32)
        a_in, b_in = a, b
    out = empty_dev(tuple(out_shape), dtype)
    ctx.binary(op, to_dev(a_in, dtype), to_dev(b_in, dtype), out, list(out_shape),
               elem_strides(sa, out_shape), elem_strides(sb, out_shape), dtype)
    ctx.check()
    got = to_host(out)
    if dtype == F32:
        assert np.array_equal(got.view(np.uint32), np.broadcast_to(want, out_shape).view(np.uint32))
    else:
        # double→float→bf16 vs fp32→bf16 can differ by one bf16 ulp on rare sums/quotients
        diff = np.abs(got.astype(np.int32) - np.broadcast_to(want, out_shape).astype(np.int32))
        assert diff.max() <= 1 and (diff != 0).mean() < 0.01
    ctx.close()
