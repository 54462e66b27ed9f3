"""The allocation-free strict forward (cfx_strict_forward_static) against the regular
entry point.

Some hosts may not allocate device memory once they run: a rollout worker embedded in a
runtime that owns the whole device heap, or a loop that cannot take cudaMalloc's device-wide
synchronisation.  For them the library keeps its scratch in one fixed device array; the caller
passes weights, state, inputs and outputs.  This file is collected last on purpose: it calls
the entry point through the C ABI twice in a row (the array keeps the previous call's
contents) and expects the outputs of cfx_policy_forward with CFX_PREC_FP32, whether it runs
alone in a fresh process or after every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
H, L, A = 256, 2, 43


def test_static_scratch_forward_matches_regular_entry_point_twice(cfx, gpu, oracle):
    n = 96
    lib = cfx.lib()
    rng = np.random.default_rng(42)
    params = oracle.init_weights(H, L, A, seed=13, scheme="uniform")
    state0 = rng.normal(0, 1, (L, n, H)).astype(np.float32)
    recs = [oracle.synthetic_records(n, seed=s) for s in (21, 22)]
    terms = [(rng.random(n) < 0.3).astype(np.float32) for _ in range(2)]
    unis = [rng.random(n, dtype=np.float32) for _ in range(2)]

    # regular entry point: two consecutive steps on a handle
    pol = cfx.Policy(n, H, L, A, "fp32")
    pol.set_weights(params)
    pol.set_state(state0)
    want = []
    for t in range(2):
        d = pol.forward_host(recs[t], terms[t], unis[t], want_r_state=True)
        want.append({k: v.copy() for k, v in d.items()})
    want_state = pol.get_state()
    pol.close()

    # allocation-free entry point: the caller owns every buffer it passes
    d_params = cfx.DeviceBuffer.from_host(params)
    d_state = cfx.DeviceBuffer.from_host(state0)
    d_rec = cfx.DeviceBuffer((n, 996), np.uint8)
    d_pt = cfx.DeviceBuffer((n,), np.float32)
    d_u = cfx.DeviceBuffer((n,), np.float32)
    out = {"env_actions": cfx.DeviceBuffer((n,), np.float32), "actions": cfx.DeviceBuffer((n,), np.int32),
           "logprobs": cfx.DeviceBuffer((n,), np.float32), "values": cfx.DeviceBuffer((n,), np.float32),
           "logits_av": cfx.DeviceBuffer((n, A + 1), np.float32),
           "r_state": cfx.DeviceBuffer((L, n, H), np.float32)}
    for t in range(2):
        d_rec.upload(recs[t])
        d_pt.upload(terms[t])
        d_u.upload(unis[t])
        io = cfx.ForwardIO(d_rec.ptr, d_pt.ptr, d_u.ptr, out["env_actions"].ptr, out["actions"].ptr,
                           out["logprobs"].ptr, out["values"].ptr, out["logits_av"].ptr,
                           out["r_state"].ptr, 0, 0, 0)
        cfx.check(lib.cfx_strict_forward_static(0, d_params.ptr, H, L, A, n, d_state.ptr, C.byref(io),
                                                None, None))
        cfx.check(lib.cfx_stream_sync(0, None))
        for k, buf in out.items():
            got = buf.download()
            if got.dtype == np.int32:
                assert np.array_equal(got, want[t][k]), (t, k)
            else:
                assert np.abs(got - want[t][k]).max() <= 2e-5, (t, k)
    assert np.abs(d_state.download() - want_state).max() <= 2e-5


def test_static_scratch_rejects_sizes_beyond_the_array(cfx, gpu):
    lib = cfx.lib()
    dummy = cfx.DeviceBuffer((64,), np.float32)
    io = cfx.ForwardIO(dummy.ptr, None, None, None, dummy.ptr, None, None, None, None, 0, 0, 0)
    for hidden, layers, n in ((256, 2, 2048), (256, 5, 64), (512, 2, 64), (256, 2, 48)):
        rc = lib.cfx_strict_forward_static(0, dummy.ptr, hidden, layers, A, n, dummy.ptr, C.byref(io),
                                           None, None)
        assert rc == 1, (hidden, layers, n)
        assert b"cfx_strict_forward_static" in lib.cfx_last_error()
    assert b"1024" in lib.cfx_last_error() or b"multiple of 32" in lib.cfx_last_error()
