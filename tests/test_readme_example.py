"""BASELINE config 1 - the reference's README example (Linear(3 -> 1) + MSE + SGD, f32, 10000 x 3) - as a
parity case: the op-by-op composition of tests/readme_example.py on the CPU oracle against float64 numpy, and
on the CUDA library against the oracle."""
import numpy as np
import pytest

import readme_example as R

STEPS = 5


def test_oracle_follows_the_float64_model(oracle):
    losses, W, b = R.train(oracle, STEPS)
    want_losses, want_W, want_b = R.train_numpy(STEPS)
    assert np.allclose(losses, want_losses, rtol=1e-4)          # f32 sums of 10000 terms in the element type
    assert np.allclose(W, want_W, rtol=1e-4, atol=1e-6) and np.allclose(b, want_b, rtol=1e-4, atol=1e-6)
    assert losses[-1] < losses[0]


@pytest.mark.gpu
def test_cuda_matches_the_oracle(oracle, cuda):
    ref_losses, ref_W, ref_b = R.train(oracle, STEPS)
    losses, W, b = R.train(cuda, STEPS)
    # reductions and dot products over 10000 f32 terms are summed in a different order: rel 1e-4
    assert np.allclose(losses, ref_losses, rtol=1e-4)
    assert np.allclose(W, ref_W, rtol=1e-4, atol=1e-6) and np.allclose(b, ref_b, rtol=1e-4, atol=1e-6)


@pytest.mark.gpu
def test_device_resident_example_matches_the_oracle(oracle, cuda):
    """maidenx_b200.readme_example keeps every tensor on the device (the form the benchmark times); same parameters
    and last loss as the oracle composition above."""
    from maidenx_b200 import device, readme_example as E
    ref_losses, ref_W, ref_b = R.train(oracle, STEPS)
    losses, W, b = E.train(E.CudaEngine(), STEPS, read_every=1)
    assert device.last_error() is None
    assert np.allclose(losses, ref_losses, rtol=1e-4)
    assert np.allclose(W, ref_W, rtol=1e-4, atol=1e-6) and np.allclose(b, ref_b, rtol=1e-4, atol=1e-6)
