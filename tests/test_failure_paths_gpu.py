"""What happens when something inside a tensor-core kernel does not arrive.

Every wait inside those kernels is bounded.  The test below makes one run out in the allowed way: the TMA producer is
told to stop early (a test hook of the C ABI), so the other roles wait for tiles that nothing will ever deliver, the
shortened limit expires, the kernel records a code and returns, and the call reports an error.  Nothing faults or hangs;
the same process then runs the same operator normally."""
import numpy as np
import pytest

from tests import datagen

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_leaves_the_context_usable():
    from superkmeans_b200 import _lib, engine

    if not engine.tensor_cores_enabled():
        pytest.skip("the tensor-core kernels are switched off")
    n, d, k = 4096, 256, 700
    x = datagen.gaussian_mixture(n, d, k, 0.3, 3)
    y = x[:k].copy()
    want, _ = engine.find_nearest(x, y)
    # about a tenth of a second at 2 GHz; the producer stops after three of the 16 k-blocks of the first tile
    _lib.check(_lib.lib.skm_debug_wait_injection(200_000_000, 3))
    try:
        with pytest.raises(RuntimeError, match="gave up waiting on a barrier"):
            engine.find_nearest(x, y)
    finally:
        _lib.check(_lib.lib.skm_debug_wait_injection(0, 0))
    got, dist = engine.find_nearest(x, y)
    np.testing.assert_array_equal(got, want)
    assert (dist >= 0).all()
