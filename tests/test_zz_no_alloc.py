"""The allocation-free strict forward (cfx_strict_forward_static) against the regular
entry point.

Some hosts may not allocate device memory once they run: a rollout worker embedded in a
runtime that owns the whole device heap, or a loop that cannot take cudaMalloc's device-wide
synchronisation.  For them the library keeps its scratch in one fixed device array; the caller
passes weights, state, inputs and outputs.  This file is collected last on purpose: it calls
the entry point through the C ABI twice in a row (the array keeps the previous call's
contents) and expects the outputs of cfx_policy_forward with CFX_PREC_FP32 bit for bit (the
two run the same kernels in the same order), whether it runs alone in a fresh process or
after every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
H, A = 256, 43


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint32) if a.dtype == np.float32 else a


def run_both(cfx, oracle, n, L, steps, use_philox):
    """`steps` consecutive forwards through both entry points on the same inputs; returns the
    per-step outputs and the final state of each."""
    lib = cfx.lib()
    rng = np.random.default_rng(42 + n + L)
    params = oracle.init_weights(H, L, A, seed=13, scheme="uniform")
    state0 = rng.normal(0, 1, (L, n, H)).astype(np.float32)
    recs = [oracle.synthetic_records(n, seed=21 + s) for s in range(steps)]
    terms = [(rng.random(n) < 0.3).astype(np.float32) for _ in range(steps)]
    unis = [None if use_philox else rng.random(n, dtype=np.float32) for _ in range(steps)]
    seed, env_offset, step0 = 77, 4096, 5

    # regular entry point: consecutive steps on a handle
    pol = cfx.Policy(n, H, L, A, "fp32")
    pol.set_weights(params)
    pol.set_state(state0)
    pol.step = step0
    want = []
    for t in range(steps):
        d = pol.forward_host(recs[t], terms[t], unis[t], seed=seed, env_offset=env_offset,
                             bump_step=True, want_r_state=True)
        want.append({k: v.copy() for k, v in d.items()})
    want_state = pol.get_state()
    pol.close()

    # allocation-free entry point: the caller owns every buffer it passes
    d_params = cfx.DeviceBuffer.from_host(params)
    d_state = cfx.DeviceBuffer.from_host(state0)
    d_rec = cfx.DeviceBuffer((n, 996), np.uint8)
    d_pt = cfx.DeviceBuffer((n,), np.float32)
    d_u = cfx.DeviceBuffer((n,), np.float32)
    d_ctr = cfx.DeviceBuffer((1,), np.uint64)
    out = {"env_actions": cfx.DeviceBuffer((n,), np.float32), "actions": cfx.DeviceBuffer((n,), np.int32),
           "logprobs": cfx.DeviceBuffer((n,), np.float32), "values": cfx.DeviceBuffer((n,), np.float32),
           "logits_av": cfx.DeviceBuffer((n, A + 1), np.float32),
           "r_state": cfx.DeviceBuffer((L, n, H), np.float32)}
    got = []
    for t in range(steps):
        d_rec.upload(recs[t])
        d_pt.upload(terms[t])
        if unis[t] is not None:
            d_u.upload(unis[t])
        d_ctr.upload(np.array([step0 + t], np.uint64))   # the caller keeps the step counter
        io = cfx.ForwardIO(d_rec.ptr, d_pt.ptr, None if use_philox else d_u.ptr, out["env_actions"].ptr,
                           out["actions"].ptr, out["logprobs"].ptr, out["values"].ptr,
                           out["logits_av"].ptr, out["r_state"].ptr, seed, env_offset, 0, 0)
        cfx.check(lib.cfx_strict_forward_static(0, d_params.ptr, H, L, A, n, d_state.ptr, C.byref(io),
                                                d_ctr.ptr, None))
        cfx.check(lib.cfx_stream_sync(0, None))
        got.append({k: buf.download() for k, buf in out.items()})
    return want, want_state, got, d_state.download()


@pytest.mark.parametrize("n,L,use_philox", [(96, 2, False), (96, 2, True), (1024, 4, False)],
                         ids=["given-uniforms", "philox-step-counter", "array-limits"])
def test_static_scratch_forward_matches_regular_entry_point_twice(cfx, gpu, oracle, n, L, use_philox):
    want, want_state, got, got_state = run_both(cfx, oracle, n, L, 2, use_philox)
    for t in range(2):   # the second call runs on the first call's leftovers in the array
        for k in got[t]:
            assert np.array_equal(bits(got[t][k]), bits(want[t][k])), (t, k)
    assert np.array_equal(bits(got_state), bits(want_state))
    if use_philox:
        # the draws are the documented Philox stream: subsequence env_offset + env, offset step
        for t in range(2):
            u = cfx.philox_uniforms(77, 4096, 5 + t, n)
            a, lp = cfx.sample_actions(got[t]["logits_av"], u, A)
            assert np.array_equal(a, got[t]["actions"])
            assert np.array_equal(bits(lp), bits(got[t]["logprobs"]))


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


def test_static_scratch_rejects_bad_pointers_and_devices_before_any_launch(cfx, gpu):
    lib = cfx.lib()
    dummy = cfx.DeviceBuffer((64,), np.float32)
    # a records pointer that is not 16-byte aligned (the encoder reads the tail floats as words)
    io = cfx.ForwardIO(dummy.ptr + 2, None, None, None, dummy.ptr, None, None, None, None, 0, 0, 0)
    rc = lib.cfx_strict_forward_static(0, dummy.ptr, 256, 2, A, 64, dummy.ptr, C.byref(io), None, None)
    assert rc == 1 and b"aligned" in lib.cfx_last_error()
    # a device ordinal that does not exist
    io = cfx.ForwardIO(dummy.ptr, None, None, None, dummy.ptr, None, None, None, None, 0, 0, 0)
    rc = lib.cfx_strict_forward_static(63, dummy.ptr, 256, 2, A, 64, dummy.ptr, C.byref(io), None, None)
    assert rc == 1 and b"device" in lib.cfx_last_error()
    # the stand-alone expand has the 4-byte form of the same rule
    out = cfx.DeviceBuffer((32, 843), np.float32)
    rc = lib.cfx_expand_obs(0, dummy.ptr + 2, out.ptr, 32, None)
    assert rc == 1 and b"aligned" in lib.cfx_last_error()
    cfx.check(lib.cfx_stream_sync(0, None))   # nothing was launched: the context is clean
