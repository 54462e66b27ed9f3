"""GPU parity tests of the fused tcgen05 kernel (fp16 / bf16 operands) through the C ABI:
against the CPU oracle on reference-env records, against the strict-fp32 device path at
multi-tile sizes, and bit-level checks of the in-kernel expand and sampler."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
H, L, A = 256, 2, 43
TOL = {"f16": 2e-2, "bf16": 1e-1}   # f16: the acceptance bound for logits/value


def _run(cfx, n, layers, prec, params, rec, prev_t, u, state, **kw):
    pol = cfx.Policy(n, H, layers, A, prec)
    pol.set_weights(params)
    pol.set_state(state)
    d = pol.forward_host(rec, prev_t, u, **kw)
    d = {k: v.copy() for k, v in d.items()}
    st = pol.get_state()
    launches = pol.last_launches
    pol.close()
    return d, st, launches


@pytest.mark.parametrize("prec", ["f16", "bf16"])
def test_fused_matches_oracle_on_env_records(cfx, gpu, oracle, golden_env, golden_oracle, prec):
    recs, terms = golden_env["records"], golden_env["prev_terminals"]
    T, n = recs.shape[:2]
    params = oracle.init_weights(H, L, A, seed=int(golden_oracle["weight_seed"]))
    pol = cfx.Policy(n, H, L, A, prec)
    pol.set_weights(params)
    st = np.zeros((L, n, H), np.float32)
    worst, agree = 0.0, 0
    for t in range(T):
        pol.set_state(st)                      # single-step protocol: same state on both sides
        d = pol.forward_host(recs[t], terms[t], golden_oracle["uniforms"][t])
        lav = oracle.forward(params, recs[t], terms[t], st, H, L, A)
        worst = max(worst, float(np.abs(d["logits_av"] - lav).max()))
        agree += int((d["logits_av"][:, :A].argmax(1) == lav[:, :A].argmax(1)).sum())
        assert np.abs(pol.get_state() - st).max() < TOL[prec]
        # the in-kernel sampler on the kernel's own logits and the given uniforms
        a, lp = cfx.sample_actions(d["logits_av"], golden_oracle["uniforms"][t])
        assert np.array_equal(a, d["actions"])
        assert np.array_equal(lp.view(np.uint32), d["logprobs"].view(np.uint32))
        assert np.array_equal(d["values"], d["logits_av"][:, A])
        assert np.array_equal(d["env_actions"], d["actions"].astype(np.float32))
    assert pol.last_launches == 1
    print(f"[{prec}] max|dlogit|={worst:.3e} greedy agreement={agree / (T * n):.4f}")
    assert worst < TOL[prec]
    if prec == "f16":
        assert agree / (T * n) >= 0.995
    pol.close()


@pytest.mark.parametrize("n,layers", [(32, 2), (96, 3), (160, 2), (416, 1), (128 * 5 + 64, 2), (288, 4)])
def test_fused_ragged_sizes(cfx, gpu, oracle, n, layers):
    rng = np.random.default_rng(n)
    rec = oracle.synthetic_records(n, seed=4)
    params = oracle.init_weights(H, layers, A, seed=5, scheme="uniform")
    state = rng.normal(0, 1, (layers, n, H)).astype(np.float32)
    prev_t = (rng.random(n) < 0.3).astype(np.float32)
    u = rng.random(n, dtype=np.float32)
    d, st, _ = _run(cfx, n, layers, "f16", params, rec, prev_t, u, state)
    want_st = state.copy()
    lav = oracle.forward(params, rec, prev_t, want_st, H, layers, A)
    assert np.abs(d["logits_av"] - lav).max() < 2e-2
    assert np.abs(st - want_st).max() < 2e-2
    assert (d["actions"] >= 0).all() and (d["actions"] < A).all()


def test_fused_many_tiles_matches_strict_path(cfx, gpu, oracle):
    """More tiles than SMs (persistent loop, ring phases wrapping) against the fp32 device path."""
    n = 148 * 128 * 2 + 5 * 128 + 32
    rng = np.random.default_rng(1)
    base = oracle.synthetic_records(4096, seed=8)
    rec = base[rng.integers(0, 4096, n)]
    params = oracle.init_weights(H, L, A, seed=6)
    state = rng.normal(0, 1, (L, n, H)).astype(np.float32)
    prev_t = (rng.random(n) < 0.05).astype(np.float32)
    d0, st0, _ = _run(cfx, n, L, "fp32", params, rec, prev_t, None, state, seed=5)
    d1, st1, launches = _run(cfx, n, L, "f16", params, rec, prev_t, None, state, seed=5)
    assert launches == 1
    # synthetic records drive every map channel over its full range, so activations and
    # logits are several times larger than on environment records: the bound is relative
    err = np.abs(d1["logits_av"] - d0["logits_av"]).max(1)
    scale = float(np.abs(d0["logits_av"]).max())
    print(f"many tiles: max|dlogit|={err.max():.3e} max|logit|={scale:.2f}")
    assert err.max() < 5e-3 * max(scale, 4.0), (err.max(), int(err.argmax()))
    assert np.abs(st1 - st0).max() < 5e-3 * max(float(np.abs(st0).max()), 4.0)
    assert (d1["logits_av"][:, :A].argmax(1) == d0["logits_av"][:, :A].argmax(1)).mean() >= 0.995
    assert (d1["actions"] == d0["actions"]).mean() > 0.98   # same Philox draws, near-equal logits
    # deterministic: a second run gives the same bits
    d2, st2, _ = _run(cfx, n, L, "f16", params, rec, prev_t, None, state, seed=5)
    assert np.array_equal(d1["logits_av"], d2["logits_av"]) and np.array_equal(st1, st2)


def test_fused_expand_is_exact_for_every_map_feature(cfx, gpu, oracle):
    """Selection weights route single features to the logits through exactly representable
    steps (zero gate weights: per layer h <- 0.125 + 0.5 h), so every one of the 792 map
    bytes of the in-kernel expand is checked bit for bit, and the 51 tail floats to fp16
    rounding."""
    n = 128
    rng = np.random.default_rng(3)
    rec = oracle.synthetic_records(n, seed=12)
    rec[:, :792] = rng.integers(0, 256, (n, 792), dtype=np.uint8)   # any byte value
    x = oracle.expand(rec)
    o = oracle.offsets(H, L, A)
    pol = cfx.Policy(n, H, L, A, "f16")
    for base in (0, 256, 512, 843 - 256):
        for u0 in range(0, H, A):
            units = np.arange(u0, min(u0 + A, H))
            params = np.zeros(o["count"], np.float32)
            params[:o["b_enc"]].reshape(843, H)[base + np.arange(H), np.arange(H)] = 1.0
            params[o["w_a"]:o["b_a"]].reshape(A, H)[np.arange(units.size), units] = 1.0
            pol.set_weights(params)
            pol.reset_state()
            d = pol.forward_host(rec, None, np.full(n, 0.5, np.float32))
            feats = base + units
            got = d["logits_av"][:, :units.size]
            want = 0.1875 + 0.25 * x[:, feats].astype(np.float64)
            is_map = feats < 792
            assert np.array_equal(got[:, is_map], want[:, is_map].astype(np.float32)), (base, u0)
            if (~is_map).any():
                assert np.abs(got[:, ~is_map] - want[:, ~is_map]).max() < 1e-3
    pol.close()


def test_fused_rejects_what_it_cannot_do(cfx, gpu, oracle):
    with pytest.raises(cfx.CfxError):
        cfx.Policy(64, 64, 2, A, "f16")         # hidden 64 is not instantiated
    with pytest.raises(cfx.CfxError):
        cfx.Policy(64, H, L, A, "tf32")         # tf32 operands are not built


def test_fused_records_r_state(cfx, gpu, oracle):
    """The optional BPTT record holds the post-zero INPUT state of every layer: the previous
    state, zeroed where prev_terminals is set - exactly, in every precision."""
    n = 128 * 3 + 64
    rng = np.random.default_rng(5)
    rec = oracle.synthetic_records(n, seed=2)
    params = oracle.init_weights(H, 3, A, seed=4)
    state = rng.normal(0, 1, (3, n, H)).astype(np.float32)
    prev_t = (rng.random(n) < 0.3).astype(np.float32)
    want = state.copy()
    want[:, prev_t != 0] = 0
    for prec in ("f16", "fp32"):
        pol = cfx.Policy(n, H, 3, A, prec)
        pol.set_weights(params)
        pol.set_state(state)
        d = pol.forward_host(rec, prev_t, None, want_r_state=True)
        assert np.array_equal(d["r_state"], want), prec
        # the bf16 record (the reference's r_state_bf16 mode): __float2bfloat16 of the same values
        pol.set_state(state)
        d = pol.forward_host(rec, prev_t, None, want_r_state="bf16")
        u = want.view(np.uint32).astype(np.uint64)
        want_bf = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
        assert d["r_state"].dtype == np.uint16 and np.array_equal(d["r_state"], want_bf), prec
        pol.close()


@pytest.mark.parametrize("n,layers", [(64, 2), (128 * 7, 2), (128 * 300 + 96, 3)])
def test_fused_single_cta_mode_equals_pair_mode(cfx, gpu, oracle, monkeypatch, n, layers):
    """The kernel runs as clusters of two CTAs (one 256-row MMA per pair) by default and as one
    CTA per tile with CFX_FUSED_PAIR=0 (read when the policy is created).  Both modes issue the
    same products in the same order for every row, so they must agree bit for bit; odd tile
    counts exercise the filler tile of the last pair."""
    rng = np.random.default_rng(n)
    base = oracle.synthetic_records(min(n, 4096), seed=9)
    rec = base[rng.integers(0, base.shape[0], n)]
    params = oracle.init_weights(H, layers, A, seed=3)
    state = rng.normal(0, 1, (layers, n, H)).astype(np.float32)
    prev_t = (rng.random(n) < 0.1).astype(np.float32)
    out = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("CFX_FUSED_PAIR", mode)
        out[mode] = _run(cfx, n, layers, "f16", params, rec, prev_t, None, state, seed=11)
    (d1, st1, _), (d0, st0, _) = out["1"], out["0"]
    assert np.array_equal(d1["logits_av"], d0["logits_av"])
    assert np.array_equal(st1, st0)
    assert np.array_equal(d1["actions"], d0["actions"])
    assert np.array_equal(d1["logprobs"], d0["logprobs"])


def test_bounded_wait_reports_a_timeout_and_leaves_the_context_usable(cfx, gpu, oracle):
    """Every wait in the kernels is bounded.  The self-test kernel waits 5 ms on a barrier that
    nothing sets, gives up and reports through the status word; afterwards a normal forward
    runs on the same context."""
    rc = cfx.lib().cfx_selftest_wait_timeout(0, 5)
    assert rc == cfx.ERR_DEVICE_TIMEOUT, cfx.lib().cfx_last_error()
    assert b"timed out" in cfx.lib().cfx_last_error()
    pol = cfx.Policy(64, H, L, A, "f16")
    pol.set_weights(oracle.init_weights(H, L, A, seed=1))
    d = pol.forward_host(oracle.synthetic_records(64, seed=1), None, None)
    assert np.isfinite(d["logits_av"]).all()
    pol.check()
    pol.close()


@pytest.mark.parametrize("prec", ["f16", "fp32"])
def test_forward_replays_from_a_cuda_graph(cfx, gpu, oracle, prec):
    """cfx_policy_forward allocates nothing, never synchronises and reads the sampler offset from
    device memory, so one captured forward (with the step bump) replays as a CUDA graph: replay k
    gives what the k-th eager forward gives (same state evolution, same Philox offsets)."""
    import torch
    n, steps = 128 * 5 + 32, 3
    rng = np.random.default_rng(8)
    rec = oracle.synthetic_records(n, seed=3)
    prev_t = (rng.random(n) < 0.1).astype(np.float32)
    pol = cfx.Policy(n, H, L, A, prec)
    pol.set_weights(oracle.init_weights(H, L, A, seed=2))
    d_rec, d_pt = cfx.DeviceBuffer.from_host(rec), cfx.DeviceBuffer.from_host(prev_t)
    d_act = cfx.DeviceBuffer((n,), np.int32)
    d_lp = cfx.DeviceBuffer((n,), np.float32)
    d_lav = cfx.DeviceBuffer((n, A + 1), np.float32)
    stream = torch.cuda.Stream()
    sp = stream.cuda_stream

    def forward():
        pol.forward_device(d_rec, d_pt, None, actions=d_act, logprobs=d_lp, logits_av=d_lav,
                           seed=9, bump_step=True, stream=sp)

    eager = []
    for _ in range(steps):
        forward()
        pol.check(sp)
        eager.append((d_act.download().copy(), d_lp.download().copy(), d_lav.download().copy()))
    assert pol.step == steps
    pol.reset_state()
    pol.step = 0
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
        forward()
    assert pol.step == 0                      # capturing runs nothing
    for k in range(steps):
        graph.replay()
        torch.cuda.synchronize()
        pol.check()
        assert np.array_equal(d_act.download(), eager[k][0]), k
        assert np.array_equal(d_lp.download().view(np.uint32), eager[k][1].view(np.uint32)), k
        assert np.array_equal(d_lav.download().view(np.uint32), eager[k][2].view(np.uint32)), k
    assert pol.step == steps
    pol.close()


@pytest.mark.parametrize("n", [65536 + 32, 65536 + 128 * 3 + 32, 32768 * 5])
def test_host_forward_in_slices_equals_one_launch(cfx, gpu, oracle, n):
    """From 65,536 envs cfx_policy_forward_host uploads the records in slices on a copy stream and
    launches the kernel per slice (a tile range) behind them.  The result must be what one launch
    over device-resident inputs gives, bit for bit, including the step bump and the r_state record."""
    rng = np.random.default_rng(n)
    base = oracle.synthetic_records(4096, seed=6)
    rec = base[rng.integers(0, 4096, n)]
    params = oracle.init_weights(H, L, A, seed=12)
    state = rng.normal(0, 1, (L, n, H)).astype(np.float32)
    prev_t = (rng.random(n) < 0.1).astype(np.float32)
    pol = cfx.Policy(n, H, L, A, "f16")
    pol.set_weights(params)
    pol.set_state(state)
    pol.step = 4
    d_rec, d_pt = cfx.DeviceBuffer.from_host(rec), cfx.DeviceBuffer.from_host(prev_t)
    d_act = cfx.DeviceBuffer((n,), np.int32)
    d_lp = cfx.DeviceBuffer((n,), np.float32)
    d_lav = cfx.DeviceBuffer((n, A + 1), np.float32)
    d_rs = cfx.DeviceBuffer((L, n, H), np.float32)
    pol.forward_device(d_rec, d_pt, None, actions=d_act, logprobs=d_lp, logits_av=d_lav, r_state=d_rs,
                       seed=3, bump_step=True)
    pol.check()
    assert pol.last_launches == 1 and pol.step == 5
    want = (d_act.download(), d_lp.download(), d_lav.download(), d_rs.download(), pol.get_state())
    pol.set_state(state)
    pol.step = 4
    d = pol.forward_host(rec, prev_t, None, seed=3, bump_step=True, want_r_state=True)
    assert pol.last_launches == max(1, min(8, n // 32768)) and pol.step == 5
    assert np.array_equal(d["actions"], want[0])
    assert np.array_equal(d["logprobs"].view(np.uint32), want[1].view(np.uint32))
    assert np.array_equal(d["logits_av"].view(np.uint32), want[2].view(np.uint32))
    assert np.array_equal(d["r_state"], want[3])
    assert np.array_equal(pol.get_state(), want[4])
    pol.close()


def test_repeated_launches_are_bit_identical(cfx, gpu, oracle):
    """The same forward launched many times over a batch large enough for every CTA to run many
    tiles gives the same bits every time.  (Guards the hand-offs between the roles of the kernel:
    an accumulator overwritten while another warpgroup still read it showed up as a few rows of
    one tile changing in about one launch out of a hundred.)"""
    n, reps = 262144, 48
    rng = np.random.default_rng(n)
    base = oracle.synthetic_records(4096, seed=6)
    rec = base[rng.integers(0, 4096, n)]
    params = oracle.init_weights(H, L, A, seed=12)
    state = rng.normal(0, 1, (L, n, H)).astype(np.float32)
    prev_t = (rng.random(n) < 0.1).astype(np.float32)
    pol = cfx.Policy(n, H, L, A, "f16")
    pol.set_weights(params)
    d_rec, d_pt = cfx.DeviceBuffer.from_host(rec), cfx.DeviceBuffer.from_host(prev_t)
    d_act = cfx.DeviceBuffer((n,), np.int32)
    d_lp = cfx.DeviceBuffer((n,), np.float32)
    d_val = cfx.DeviceBuffer((n,), np.float32)
    first = None
    for rep in range(reps):
        pol.set_state(state)
        pol.step = 4
        pol.forward_device(d_rec, d_pt, None, actions=d_act, logprobs=d_lp, values=d_val, seed=3, bump_step=True)
        pol.check()
        got = (d_act.download(), d_lp.download().view(np.uint32), d_val.download().view(np.uint32))
        if first is None:
            first = got
        else:
            for name, a, b in zip(("actions", "logprobs", "values"), got, first):
                bad = np.nonzero(a != b)[0]
                assert bad.size == 0, (rep, name, bad.size, bad[:8])
    pol.close()


def test_logits_rows_in_an_array_that_is_only_16_byte_aligned(cfx, gpu, oracle):
    """logits_av need only be 16-byte aligned.  The kernel writes a 176-byte row as five 32-byte
    stores and one 16-byte store, placed by the row's own address; an array that starts 16
    bytes into an allocation swaps the roles of the even and the odd rows and must give the
    same rows, with nothing written outside them."""
    n = 288   # ragged: the last tile has 32 rows
    rng = np.random.default_rng(5)
    rec = oracle.synthetic_records(n, seed=8)
    params = oracle.init_weights(H, L, A, seed=3)
    state = rng.normal(0, 1, (L, n, H)).astype(np.float32)
    u = rng.random(n, dtype=np.float32)
    pol = cfx.Policy(n, H, L, A, "f16")
    pol.set_weights(params)
    d_rec, d_u = cfx.DeviceBuffer.from_host(rec), cfx.DeviceBuffer.from_host(u)
    d_act = cfx.DeviceBuffer((n,), np.int32)
    rows = {}
    for shift in (0, 4):   # floats: 0 and 16 bytes
        guard = np.full(n * (A + 1) + 8, -7.5, np.float32)
        d_all = cfx.DeviceBuffer.from_host(guard)

        class View:   # a DeviceBuffer-like view that starts `shift` floats into the allocation
            ptr = d_all.ptr + 4 * shift
        pol.set_state(state)
        pol.forward_device(d_rec, None, d_u, actions=d_act, logits_av=View, seed=1)
        pol.check()
        back = d_all.download()
        assert np.all(back[:shift] == -7.5) and np.all(back[shift + n * (A + 1):] == -7.5)
        rows[shift] = back[shift:shift + n * (A + 1)].reshape(n, A + 1).copy()
    assert np.array_equal(rows[0].view(np.uint32), rows[4].view(np.uint32))
    assert np.all(rows[0] != -7.5)
    pol.close()
