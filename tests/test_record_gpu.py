"""Record write (cfx_record_obs) against its numpy restatement (oracle.record_from_state), and
the restatement against the reference's own kernel on the reference's own device state."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,seed", [(32, 1), (2048 + 96, 2)])
def test_record_write_matches_the_oracle_on_synthetic_state(cfx, gpu, oracle, n, seed):
    st = oracle.synthetic_env_state(n, seed=seed)
    want = oracle.record_from_state(st)
    view, keep = cfx.env_view_from_state(st)
    d_rec = cfx.DeviceBuffer.from_host(np.full((n, 996), 0xCD, np.uint8))
    cfx.record_obs(view, d_rec)
    cfx.check(cfx.lib().cfx_stream_sync(0, None))
    got = d_rec.download()
    assert np.array_equal(got, want)
    assert (want[:, :792].reshape(n, 99, 8)[:, :, 3:] != 0).any(axis=(1, 2)).mean() > 0.5   # mobs in most views

    # skip flags: flagged rows keep their bytes
    skip = (np.arange(n) % 3 == 0).astype(np.uint8)
    d_rec2 = cfx.DeviceBuffer.from_host(np.full((n, 996), 0xCD, np.uint8))
    cfx.record_obs(view, d_rec2, skip=cfx.DeviceBuffer.from_host(skip))
    cfx.check(cfx.lib().cfx_stream_sync(0, None))
    got2 = d_rec2.download()
    assert np.array_equal(got2[skip == 0], want[skip == 0]) and np.all(got2[skip == 1] == 0xCD)

    # list variant: 12-byte entries whose first int32 is the env; entries out of range are ignored
    envs = np.array([n - 1, 0, 5, n // 2, -1, n], np.int32)
    lst = np.zeros((envs.size, 3), np.int32)
    lst[:, 0] = envs
    lst[:, 1:] = 0x5A5A5A5A
    d_rec3 = cfx.DeviceBuffer.from_host(np.full((n, 996), 0xCD, np.uint8))
    cfx.record_obs_list(view, d_rec3, cfx.DeviceBuffer.from_host(lst), 12,
                        cfx.DeviceBuffer.from_host(np.array([envs.size], np.int32)))
    cfx.check(cfx.lib().cfx_stream_sync(0, None))
    got3 = d_rec3.download()
    listed = np.zeros(n, bool)
    listed[envs[(envs >= 0) & (envs < n)]] = True
    assert np.array_equal(got3[listed], want[listed]) and np.all(got3[~listed] == 0xCD)
    del keep


@pytest.mark.parametrize("fuzz", [0, 2], ids=["random-play", "randomised-state"])
def test_record_oracle_equals_the_reference_kernel_on_its_own_state(cfx, gpu, oracle, fuzz):
    """The numpy restatement reads the reference's live device state through the view the
    binding fills and reproduces what k_record_obs wrote for it (craftax_full.cu:9180-9297)."""
    if not oracle.RefCuda.available(2):
        pytest.skip("oracle/_ref/libcfref_cuda_l2.so not built (reference sources absent)")
    cfx.lib()
    n = 512
    view = cfx.EnvView()
    ref = oracle.RefCuda.record_session(2, n, 64, fuzz, 9, view)
    try:
        st = cfx.env_state_from_view(view)
        d_rec = cfx.DeviceBuffer((n, 996), np.uint8)
        cfx.record_obs(view, d_rec)
        cfx.check(cfx.lib().cfx_stream_sync(0, None))
        got = d_rec.download()
    finally:
        oracle.RefCuda.record_session_close(2)
    assert np.array_equal(oracle.record_from_state(st), ref)
    assert np.array_equal(got, ref)
