"""Both launches of a two-launch plan as one persistent kernel (tfft_plan_fuse_launches): the
arithmetic is that of the two launches, so the outputs must be bit-identical, for whole and
ragged chunk counts, every lag, repeated execs and the inverse direction."""
import pytest

torch = pytest.importorskip("torch")
pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a CUDA device")]


@pytest.mark.parametrize("logn,dtype", [(15, 0), (16, 0), (16, 1)])
@pytest.mark.parametrize("batch,log_chunk,lag", [(1, 0, 0), (5, 1, 1), (37, 2, 1), (64, 3, 2), (300, 4, 1), (1024, 5, 0)])
def test_fused_launches_equal_the_two_launches(logn, dtype, batch, log_chunk, lag):
    import turbofft_b200 as tf
    torch.manual_seed(logn * 1000 + batch)
    x = torch.randn(batch << logn, dtype=torch.complex64 if dtype == 0 else torch.complex128, device="cuda")
    ref = torch.empty_like(x)
    y = torch.empty_like(x)
    stream = torch.cuda.current_stream().cuda_stream
    p = tf.Plan(logn, batch, dtype)
    p.exec_ptr(x.data_ptr(), ref.data_ptr(), stream)
    q = tf.Plan(logn, batch, dtype)
    q.fuse_launches(log_chunk, lag)
    for _ in range(3):  # the per-chunk counters are cleared by every exec
        y.zero_()
        q.exec_ptr(x.data_ptr(), y.data_ptr(), stream)
        torch.cuda.synchronize()
        assert q.device_status() == 0
        assert torch.equal(torch.view_as_real(y), torch.view_as_real(ref))
    p.destroy()
    q.destroy()


def test_fused_launches_against_float64_fft_and_inverse():
    import turbofft_b200 as tf
    logn, batch = 16, 48
    torch.manual_seed(7)
    x = torch.randn(batch, 1 << logn, dtype=torch.complex64, device="cuda")
    q = tf.Plan(logn, batch, tf.FLOAT2)
    q.fuse_launches(2, 1)
    y = q(x)
    want = torch.fft.fft(x.to(torch.complex128), dim=1)
    rel = (torch.linalg.vector_norm(y.to(torch.complex128) - want) / torch.linalg.vector_norm(want)).item()
    assert rel <= 1e-6 * logn, rel  # the tolerance of the complex64 parity tests
    q.set_direction(inverse=True, scale=1.0 / (1 << logn))
    back = q(y)
    rel = (torch.linalg.vector_norm(back - x) / torch.linalg.vector_norm(x)).item()
    assert rel <= 2e-6 * logn, rel
    assert q.device_status() == 0
    q.destroy()


def test_fused_launches_refuses_other_plans():
    import turbofft_b200 as tf
    for kwargs in (dict(logN=10, batch=64), dict(logN=16, batch=8, if_ft=1), dict(logN=22, batch=2)):
        p = tf.Plan(dtype=tf.FLOAT2, **kwargs)
        with pytest.raises(tf.TurboFFTError):
            p.fuse_launches(2, 1)
        p.destroy()
    p = tf.Plan(16, 8, tf.FLOAT2)
    with pytest.raises(tf.TurboFFTError):
        p.fuse_launches(2, 3)  # lag must stay below the ring's four chunks minus one
    p.destroy()
