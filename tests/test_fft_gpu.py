"""Fused pencil transposes: element-exact against slicing/permuting the full array, and a full 3-D FFT."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [24, 50])
def test_transposes_and_fft_single_gpu(n):
    from rbruck_alltoallv_b200.ops.fft import PencilTranspose
    from rbruck_alltoallv_b200.parallel.comm import Communicator
    comm = Communicator(nranks=1, heap_bytes=64 << 20, arena_bytes=1 << 20)
    try:
        tp = PencilTranspose(comm, n, 1, 1, seed=n)
        full = torch.view_as_complex(torch.randn(n, n, n, 2, device="cuda"))
        xp = tp.local_x_pencil_of(full)
        y = tp.x_to_y(xp)
        torch.cuda.synchronize()
        assert torch.equal(y, tp.expected_y(full))
        z = tp.y_to_z(y.clone())
        torch.cuda.synchronize()
        assert torch.equal(z, tp.expected_z(full))
        fx = torch.fft.fft(xp, dim=2)
        fy = torch.fft.fft(tp.x_to_y(fx.contiguous()), dim=2)
        fz = torch.fft.fft(tp.y_to_z(fy.contiguous()), dim=2)
        want = tp.expected_z(torch.fft.fftn(full))
        assert (fz - want).abs().max().item() <= 1e-4 * want.abs().max().item()
        tp.check()
    finally:
        comm.close()


def test_other_element_sizes():
    from rbruck_alltoallv_b200.ops.fft import PencilTranspose
    from rbruck_alltoallv_b200.parallel.comm import Communicator
    comm = Communicator(nranks=1, heap_bytes=64 << 20, arena_bytes=1 << 20)
    try:
        for dt in (torch.float32, torch.complex128):
            tp = PencilTranspose(comm, 40, 1, 1, dtype=dt, seed=3)
            full = torch.randn(40, 40, 40, device="cuda").to(dt)
            y = tp.x_to_y(tp.local_x_pencil_of(full))
            torch.cuda.synchronize()
            assert torch.equal(y, tp.expected_y(full))
    finally:
        comm.close()
